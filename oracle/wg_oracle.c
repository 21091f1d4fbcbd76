/*
 * CPU oracle for the Winograd-ReLU F(2x2,3x3) layer math.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's four GPU ops so
 * that the CUDA kernels of this repository can be checked against it.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline / reference arm may build,
 * load or call it; the product library never does.
 *
 * Parity status: pinned.  The restatement is checked (a) against the reference's own
 * known-answer structure, "Winograd layer with G g G^T weights == 3x3 SAME convolution"
 * (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_test.py:8-25,179-192),
 * (b) against autodiff of that graph for the two gradient ops
 * (winograd2x2_cublas/winograd2x2_conv/winograd2x2_conv_grad_test.py:205-227,
 *  winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_grad_test.py:194-216), and
 * (c) against outputs of the reference's own CUDA kernels compiled unmodified for
 * sm_100a (oracle/Makefile, target "ref") and run on a B200; those outputs are the fixtures under
 * tests/golden/.
 *
 * Layouts are the reference's: X (B,H,W,C); V (16,B,nH,nW,C); W (16,C,K);
 * Y (B,outH,outW,K); nH=(H+1)/2, nW=(W+1)/2; Winograd position t = 4*row + col.
 *
 * The file is compiled twice: -DREAL=float -DSUF=_f32 and -DREAL=double -DSUF=_f64.
 */
#include <omp.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL float
#define SUF _f32
#endif
#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

#ifndef WGO_THREADS_DEFINED
#define WGO_THREADS_DEFINED
/* Number of OpenMP threads the loops below use (launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1, which would silently turn the timed CPU baseline into a one-core run). */
#if defined(WGO_EXPORT_THREADS)
void wgo_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int wgo_get_max_threads(void) { return omp_get_max_threads(); }
#endif
#endif

/* B^T of F(2x2,3x3); the 16 sums at
 * winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_cuda.cu.cc:112-127
 * are (B^T d B)[i][j] = sum_{y,x} BT[i][y] BT[j][x] d[y][x] with this matrix. */
static const int BT[4][4] = {{1, 0, -1, 0}, {0, 1, 1, 0}, {0, -1, 1, 0}, {0, 1, 0, -1}};
/* A^T; the four sums at winograd2x2_cublas/winograd2x2_conv/winograd2x2_conv_cuda.cu.cc:39-46
 * are (A^T m A)[a][e] = sum_{i,j} AT[a][i] AT[e][j] m[i][j]. */
static const int AT[2][4] = {{1, 1, 1, 0}, {0, 1, -1, -1}};

/*
 * Input transform, optionally followed by the Winograd-domain ReLU.
 * Follows Winograd2x2ImTransCompute
 * (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_cuda.cu.cc:11-149):
 * 4x4 patch at (2*th-1, 2*tw-1) with zero fill outside the image (:45-92), V = B^T d B
 * (:112-127), plane stride B*nH*nW*C (:130-148).  relu!=0 applies max(0,.) as the layer
 * wrapper does with nl=tf.nn.relu (ResNet-18-var/winograd_imtrans.py:16-17).
 */
void FN(wgo_imtrans_fwd)(const REAL *X, REAL *V, int B, int H, int W, int C, int relu)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const size_t plane = (size_t)B * nH * nW * C;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int th = 0; th < nH; ++th)
            for (int tw = 0; tw < nW; ++tw) {
                const size_t off = (((size_t)b * nH + th) * nW + tw) * C;
                for (int c = 0; c < C; ++c) {
                    REAL d[4][4], r[4][4];
                    for (int y = 0; y < 4; ++y)
                        for (int x = 0; x < 4; ++x) {
                            const int fy = 2 * th - 1 + y, fx = 2 * tw - 1 + x;
                            d[y][x] = (fy >= 0 && fy < H && fx >= 0 && fx < W)
                                          ? X[(((size_t)b * H + fy) * W + fx) * C + c]
                                          : (REAL)0;
                        }
                    for (int i = 0; i < 4; ++i)
                        for (int x = 0; x < 4; ++x) {
                            REAL s = 0;
                            for (int y = 0; y < 4; ++y) s += (REAL)BT[i][y] * d[y][x];
                            r[i][x] = s;
                        }
                    for (int i = 0; i < 4; ++i)
                        for (int j = 0; j < 4; ++j) {
                            REAL s = 0;
                            for (int x = 0; x < 4; ++x) s += (REAL)BT[j][x] * r[i][x];
                            if (relu && s < 0) s = 0;
                            V[(size_t)(4 * i + j) * plane + off + c] = s;
                        }
                }
            }
}

/* M_t[P x K] = V_t[P x C] . W_t[C x K], the 16 GEMMs of
 * winograd2x2_cublas/winograd2x2_conv/winograd2x2_conv_cuda.cu.cc:80-85 (row-major view
 * of the column-major cublasSgemmBatched(N,N, m=K, n=P, k=C) call). */
static void gemm_nn(const REAL *A, const REAL *Bm, REAL *Cm, size_t P, int C, int K)
{
#pragma omp parallel for schedule(static)
    for (size_t p = 0; p < P; ++p) {
        REAL *out = Cm + p * K;
        for (int k = 0; k < K; ++k) out[k] = 0;
        for (int c = 0; c < C; ++c) {
            const REAL a = A[p * C + c];
            const REAL *w = Bm + (size_t)c * K;
            for (int k = 0; k < K; ++k) out[k] += a * w[k];
        }
    }
}

/*
 * Winograd-domain product and output transform.
 * Follows Winograd2x2ConvComputeLauncher
 * (winograd2x2_cublas/winograd2x2_conv/winograd2x2_conv_cuda.cu.cc:65-93): 16 GEMMs
 * (:80-85) into a scratch M of 16*P*K values, then Output_transform (:13-53),
 * Y[b,2th+a,2tw+e,k] = (A^T m A)[a][e].  The reference always emits 2nH x 2nW pixels
 * (winograd2x2_conv_op.cc:53); outH/outW <= 2nH/2nW crop the result the way the
 * reference's test graph does for odd sizes (winograd2x2_imTrans_test.py:152-153).
 * scratch holds 16*P*K REALs, P = B*nH*nW.
 */
void FN(wgo_conv_fwd)(const REAL *V, const REAL *Wt, REAL *Y, REAL *scratch, int B, int nH, int nW,
                      int C, int K, int outH, int outW)
{
    const size_t P = (size_t)B * nH * nW;
    for (int t = 0; t < 16; ++t)
        gemm_nn(V + (size_t)t * P * C, Wt + (size_t)t * C * K, scratch + (size_t)t * P * K, P, C, K);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int th = 0; th < nH; ++th)
            for (int tw = 0; tw < nW; ++tw) {
                const size_t p = ((size_t)b * nH + th) * nW + tw;
                for (int k = 0; k < K; ++k) {
                    REAL m[16];
                    for (int t = 0; t < 16; ++t) m[t] = scratch[((size_t)t * P + p) * K + k];
                    for (int a = 0; a < 2; ++a)
                        for (int e = 0; e < 2; ++e) {
                            const int h = 2 * th + a, w = 2 * tw + e;
                            if (h >= outH || w >= outW) continue;
                            REAL s = 0;
                            for (int i = 0; i < 4; ++i)
                                for (int j = 0; j < 4; ++j)
                                    s += (REAL)(AT[a][i] * AT[e][j]) * m[4 * i + j];
                            Y[(((size_t)b * outH + h) * outW + w) * K + k] = s;
                        }
                }
            }
}

/*
 * Gradient of the product/output-transform op.
 * Follows Winograd2x2ConvGradComputeLauncher
 * (winograd2x2_cublas/winograd2x2_conv/winograd2x2_conv_grad_cuda.cu.cc:79-124):
 * dM = A dY A^T per 2x2 block (:22-43), dV_t = dM_t . W_t^T (:103-108),
 * dW_t = V_t^T . dM_t (:115-120).  dY is (B,H,W,K); rows/columns of the 2nH x 2nW tile
 * grid beyond H/W count as zero (the reference reads them unguarded, which is only
 * defined for even sizes).  mask (16*C*K, may be NULL) multiplies dW, which is what
 * autodiff of W*mask yields (ResNet-18-var/winograd_conv.py:23-26).
 * scratch holds 16*P*K REALs.
 */
void FN(wgo_conv_bwd)(const REAL *V, const REAL *Wt, const REAL *dY, const REAL *mask, REAL *dV,
                      REAL *dW, REAL *scratch, int B, int H, int W, int C, int K)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const size_t P = (size_t)B * nH * nW;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int th = 0; th < nH; ++th)
            for (int tw = 0; tw < nW; ++tw) {
                const size_t p = ((size_t)b * nH + th) * nW + tw;
                for (int k = 0; k < K; ++k) {
                    REAL g[2][2];
                    for (int a = 0; a < 2; ++a)
                        for (int e = 0; e < 2; ++e) {
                            const int h = 2 * th + a, w = 2 * tw + e;
                            g[a][e] = (h < H && w < W) ? dY[(((size_t)b * H + h) * W + w) * K + k]
                                                       : (REAL)0;
                        }
                    for (int i = 0; i < 4; ++i)
                        for (int j = 0; j < 4; ++j) {
                            REAL s = 0;
                            for (int a = 0; a < 2; ++a)
                                for (int e = 0; e < 2; ++e)
                                    s += (REAL)(AT[a][i] * AT[e][j]) * g[a][e];
                            scratch[((size_t)(4 * i + j) * P + p) * K + k] = s;
                        }
                }
            }
    if (dV) {
#pragma omp parallel for collapse(2) schedule(static)
        for (int t = 0; t < 16; ++t)
            for (size_t p = 0; p < P; ++p) {
                const REAL *dm = scratch + ((size_t)t * P + p) * K;
                for (int c = 0; c < C; ++c) {
                    const REAL *w = Wt + ((size_t)t * C + c) * K;
                    REAL s = 0;
                    for (int k = 0; k < K; ++k) s += dm[k] * w[k];
                    dV[((size_t)t * P + p) * C + c] = s;
                }
            }
    }
    if (dW) {
#pragma omp parallel for collapse(2) schedule(static)
        for (int t = 0; t < 16; ++t)
            for (int c = 0; c < C; ++c) {
                REAL *out = dW + ((size_t)t * C + c) * K;
                for (int k = 0; k < K; ++k) out[k] = 0;
                for (size_t p = 0; p < P; ++p) {
                    const REAL v = V[((size_t)t * P + p) * C + c];
                    const REAL *dm = scratch + ((size_t)t * P + p) * K;
                    for (int k = 0; k < K; ++k) out[k] += v * dm[k];
                }
                if (mask) {
                    const REAL *mk = mask + ((size_t)t * C + c) * K;
                    for (int k = 0; k < K; ++k) out[k] *= mk[k];
                }
            }
    }
}

/*
 * Gradient of the input transform.
 * Follows Winograd2x2ImTransGradComputeLauncher
 * (winograd2x2_cublas/winograd2x2_imTrans/winograd2x2_imTrans_grad_cuda.cu.cc:118-129):
 * G = B g B^T per tile (:39-62, done here out of place; the reference overwrites its
 * input), then the overlap-add gather dX[b,h,w,c] = sum over the tiles covering (h,w) of
 * G[h+1-2th][w+1-2tw] (:98-115).  Vmask (same shape as dV, may be NULL): where
 * Vmask<=0 the incoming gradient counts as zero, i.e. the ReluGrad that autodiff of
 * nl=tf.nn.relu inserts (ResNet-18-var/winograd_imtrans.py:17).  H, W are the true
 * image sizes (the reference op assumes H=2nH, W=2nW,
 * winograd2x2_imTrans_grad_op.cc:45-46).
 */
void FN(wgo_imtrans_bwd)(const REAL *dV, const REAL *Vmask, REAL *dX, int B, int H, int W, int C)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const size_t plane = (size_t)B * nH * nW * C;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < H; ++h)
            for (int w = 0; w < W; ++w)
                for (int c = 0; c < C; ++c) {
                    REAL val = 0;
                    for (int th = 0; th < nH; ++th) {
                        const int y = h + 1 - 2 * th;
                        if (y < 0 || y > 3) continue;
                        for (int tw = 0; tw < nW; ++tw) {
                            const int x = w + 1 - 2 * tw;
                            if (x < 0 || x > 3) continue;
                            const size_t off = (((size_t)b * nH + th) * nW + tw) * C + c;
                            /* G[y][x] = sum_{i,j} BT[i][y] BT[j][x] g[i][j] */
                            REAL s = 0;
                            for (int i = 0; i < 4; ++i)
                                for (int j = 0; j < 4; ++j) {
                                    const int cf = BT[i][y] * BT[j][x];
                                    if (!cf) continue;
                                    const size_t idx = (size_t)(4 * i + j) * plane + off;
                                    REAL g = dV[idx];
                                    if (Vmask && !(Vmask[idx] > 0)) g = 0;
                                    s += (REAL)cf * g;
                                }
                            val += s;
                        }
                    }
                    dX[(((size_t)b * H + h) * W + w) * C + c] = val;
                }
}

/*
 * One whole Winograd-ReLU layer forward, X -> Y: the call sequence of
 * ResNet-18-var/imagenet-resnet-transWino-prune.py:118-119 (WinogradImTrans with
 * nl=relu, then WinogradConv).  Vbuf holds 16*P*C and scratch 16*P*K REALs.
 * This is what the benchmark times as the CPU baseline.
 */
void FN(wgo_layer_fwd)(const REAL *X, const REAL *Wt, REAL *Y, REAL *Vbuf, REAL *scratch, int B, int H,
                       int W, int C, int K, int relu)
{
    FN(wgo_imtrans_fwd)(X, Vbuf, B, H, W, C, relu);
    FN(wgo_conv_fwd)(Vbuf, Wt, Y, scratch, B, (H + 1) / 2, (W + 1) / 2, C, K, H, W);
}
