// FP32 (FFMA, CUDA-core) kernels of the Winograd-domain product: the exact-arithmetic path
// (max rel err <= 1e-5 against float64) that the tensor-core path is validated against.
//
// All three kernels walk the 16 Winograd positions one row (i = 0..3, four positions j) at a
// time, so the small A^T / A transforms fold into the kernel and no product tensor M or dM
// (16*P*K floats in the reference) is ever written to memory:
//   conv_fwd_ffma : Y  = A^T (V_t . W_t) A         tile 64 tiles x 64 out-channels
//   conv_dv_ffma  : dV_t = (A dY A^T)_t . W_t^T     tile 64 tiles x 64 in-channels
//   conv_dw_ffma  : dW_t = V_t^T . (A dY A^T)_t     tile 64 x 64 channels, split over P
#include "wg_common.cuh"

namespace wg {

constexpr int kTP = 64;   // tiles (rows of the per-position GEMM) per CTA
constexpr int kTN = 64;   // channels (columns) per CTA
constexpr int kCh = 16;   // contraction chunk held in shared memory

static __device__ __forceinline__ void decode_tile(long long p, int nH, int nW, int &b, int &th, int &tw)
{
    tw = (int)(p % nW);
    th = (int)((p / nW) % nH);
    b = (int)(p / ((long long)nW * nH));
}

// index of image-like tensor element (b, h, w, ch) for a tensor with `Cn` channels
template <int LAYOUT>
static __device__ __forceinline__ long long img_index(int b, int h, int w, int ch, int Hh, int Ww, int Cn)
{
    return LAYOUT == WG2X2_NHWC ? (((long long)b * Hh + h) * Ww + w) * Cn + ch
                                : (((long long)b * Cn + ch) * Hh + h) * Ww + w;
}

// ------------------------------------------------------------------------------------------
// Forward
// ------------------------------------------------------------------------------------------
template <bool VEC, int LAYOUT>
__global__ void __launch_bounds__(256) conv_fwd_ffma_kernel(const float *__restrict__ V, const float *__restrict__ Wt,
                                                              float *__restrict__ Y, long long P, int nH, int nW, int C, int K,
                                                              int outH, int outW)
{
    __shared__ __align__(16) float Vs[4][kCh][kTP];
    __shared__ __align__(16) float Ws[4][kCh][kTN];
    const int tid = threadIdx.x;
    const int tp = tid & 15, tk = tid >> 4;
    const long long p0 = (long long)blockIdx.x * kTP;
    const int k0 = blockIdx.y * kTN;

    float y[4][4][2][2];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) { y[a][b][0][0] = y[a][b][0][1] = y[a][b][1][0] = y[a][b][1][1] = 0.f; }

#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
        float acc[4][4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[j][a][b] = 0.f;

#pragma unroll 1
        for (int c0 = 0; c0 < C; c0 += kCh) {
            __syncthreads();
            if (VEC) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    {   // V_t[p0+pp][c0 + 4*c4 .. +3] -> Vs[j][cc][pp]
                        const int c4 = tid & 3, pp = tid >> 2;
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (p0 + pp < P && c0 + 4 * c4 < C)
                            v = __ldg(reinterpret_cast<const float4 *>(V + ((long long)(4 * i + j) * P + p0 + pp) * C + c0 + 4 * c4));
                        Vs[j][4 * c4 + 0][pp] = v.x; Vs[j][4 * c4 + 1][pp] = v.y;
                        Vs[j][4 * c4 + 2][pp] = v.z; Vs[j][4 * c4 + 3][pp] = v.w;
                    }
                    {   // W_t[c0+cc][k0 + 4*k4 .. +3] -> Ws[j][cc][..]
                        const int k4 = tid & 15, cc = tid >> 4;
                        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (c0 + cc < C && k0 + 4 * k4 < K)
                            w = __ldg(reinterpret_cast<const float4 *>(Wt + ((long long)(4 * i + j) * C + c0 + cc) * K + k0 + 4 * k4));
                        *reinterpret_cast<float4 *>(&Ws[j][cc][4 * k4]) = w;
                    }
                }
            } else {
#pragma unroll 1
                for (int e = tid; e < 4 * kCh * kTP; e += 256) {
                    const int cc = e % kCh, pp = (e / kCh) % kTP, j = e / (kCh * kTP);
                    float v = 0.f;
                    if (p0 + pp < P && c0 + cc < C) v = __ldg(V + ((long long)(4 * i + j) * P + p0 + pp) * C + c0 + cc);
                    Vs[j][cc][pp] = v;
                }
#pragma unroll 1
                for (int e = tid; e < 4 * kCh * kTN; e += 256) {
                    const int kk = e % kTN, cc = (e / kTN) % kCh, j = e / (kCh * kTN);
                    float w = 0.f;
                    if (c0 + cc < C && k0 + kk < K) w = __ldg(Wt + ((long long)(4 * i + j) * C + c0 + cc) * K + k0 + kk);
                    Ws[j][cc][kk] = w;
                }
            }
            __syncthreads();
#pragma unroll
            for (int cc = 0; cc < kCh; ++cc) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = *reinterpret_cast<const float4 *>(&Vs[j][cc][4 * tp]);
                    const float4 w = *reinterpret_cast<const float4 *>(&Ws[j][cc][4 * tk]);
                    const float av[4] = {a.x, a.y, a.z, a.w};
                    const float wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi)
#pragma unroll
                        for (int ki = 0; ki < 4; ++ki) acc[j][pi][ki] = fmaf(av[pi], wv[ki], acc[j][pi][ki]);
                }
            }
        }
        // fold Winograd row i into the 2x2 outputs
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
#pragma unroll
            for (int ki = 0; ki < 4; ++ki) {
                float z0, z1;
                at_cols(acc[0][pi][ki], acc[1][pi][ki], acc[2][pi][ki], acc[3][pi][ki], z0, z1);
                at_rows_accum(i, z0, z1, y[pi][ki]);
            }
    }

#pragma unroll
    for (int pi = 0; pi < 4; ++pi) {
        const long long p = p0 + 4 * tp + pi;
        if (p >= P) continue;
        int b, th, tw;
        decode_tile(p, nH, nW, b, th, tw);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = 2 * th + a, w = 2 * tw + e;
                if (h >= outH || w >= outW) continue;
                const int k = k0 + 4 * tk;
                if (LAYOUT == WG2X2_NHWC && VEC) {
                    if (k < K)
                        *reinterpret_cast<float4 *>(Y + img_index<LAYOUT>(b, h, w, k, outH, outW, K)) =
                            make_float4(y[pi][0][a][e], y[pi][1][a][e], y[pi][2][a][e], y[pi][3][a][e]);
                } else {
#pragma unroll
                    for (int ki = 0; ki < 4; ++ki)
                        if (k + ki < K) Y[img_index<LAYOUT>(b, h, w, k + ki, outH, outW, K)] = y[pi][ki][a][e];
                }
            }
    }
}

// ------------------------------------------------------------------------------------------
// dM producer shared by the two gradient kernels: Winograd row i of A dY A^T for tile p and
// output channel k, with out-of-image gradient taken as zero.
// ------------------------------------------------------------------------------------------
template <int LAYOUT>
static __device__ __forceinline__ void load_dy_block(const float *__restrict__ dY, long long p, int k, int nH, int nW,
                                                     int H, int W, int K, float (&g)[2][2])
{
    int b, th, tw;
    decode_tile(p, nH, nW, b, th, tw);
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int h = 2 * th + a, w = 2 * tw + e;
            g[a][e] = (h < H && w < W) ? __ldg(dY + img_index<LAYOUT>(b, h, w, k, H, W, K)) : 0.f;
        }
}

// ------------------------------------------------------------------------------------------
// dV_t[p][c] = sum_k dM_t[p][k] W_t[c][k]   (optionally zeroed where the saved V <= 0)
// ------------------------------------------------------------------------------------------
template <int LAYOUT>
__global__ void __launch_bounds__(256) conv_dv_ffma_kernel(const float *__restrict__ Vsaved, const float *__restrict__ Wt,
                                                             const float *__restrict__ dY, float *__restrict__ dV, long long P,
                                                             int nH, int nW, int H, int W, int C, int K, int relu)
{
    __shared__ __align__(16) float Ms[4][kCh][kTP];   // dM rows, [j][kk][pp]
    __shared__ __align__(16) float Ws[4][kCh][kTN];   // W^T,    [j][kk][cc]
    const int tid = threadIdx.x;
    const int tp = tid & 15, tc = tid >> 4;
    const long long p0 = (long long)blockIdx.x * kTP;
    const int c0 = blockIdx.y * kTN;

#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
        float acc[4][4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[j][a][b] = 0.f;
#pragma unroll 1
        for (int k0 = 0; k0 < K; k0 += kCh) {
            __syncthreads();
            // dM: 64 tiles x 16 k = 1024 (tile,k) pairs, 4 per thread
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int e = tid + 256 * r;
                // NHWC: k fastest (contiguous in dY); NCHW: tile fastest (w contiguous in dY)
                const int kk = LAYOUT == WG2X2_NHWC ? (e % kCh) : (e / kTP);
                const int pp = LAYOUT == WG2X2_NHWC ? (e / kCh) : (e % kTP);
                float dm[4] = {0.f, 0.f, 0.f, 0.f};
                if (p0 + pp < P && k0 + kk < K) {
                    float g[2][2];
                    load_dy_block<LAYOUT>(dY, p0 + pp, k0 + kk, nH, nW, H, W, K, g);
                    a_g_at_row(i, g[0][0], g[0][1], g[1][0], g[1][1], dm);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) Ms[j][kk][pp] = dm[j];
            }
            // W_t[c0+cc][k0+kk] -> Ws[j][kk][cc]
#pragma unroll 1
            for (int e = tid; e < 4 * kCh * kTN; e += 256) {
                const int kk = e % kCh, cc = (e / kCh) % kTN, j = e / (kCh * kTN);
                float w = 0.f;
                if (c0 + cc < C && k0 + kk < K) w = __ldg(Wt + ((long long)(4 * i + j) * C + c0 + cc) * K + k0 + kk);
                Ws[j][kk][cc] = w;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kCh; ++kk) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = *reinterpret_cast<const float4 *>(&Ms[j][kk][4 * tp]);
                    const float4 w = *reinterpret_cast<const float4 *>(&Ws[j][kk][4 * tc]);
                    const float av[4] = {a.x, a.y, a.z, a.w};
                    const float wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi)
#pragma unroll
                        for (int ci = 0; ci < 4; ++ci) acc[j][pi][ci] = fmaf(av[pi], wv[ci], acc[j][pi][ci]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int pi = 0; pi < 4; ++pi) {
                const long long p = p0 + 4 * tp + pi;
                if (p >= P) continue;
#pragma unroll
                for (int ci = 0; ci < 4; ++ci) {
                    const int c = c0 + 4 * tc + ci;
                    if (c >= C) continue;
                    const long long idx = ((long long)(4 * i + j) * P + p) * C + c;
                    float v = acc[j][pi][ci];
                    if (relu && !(__ldg(Vsaved + idx) > 0.f)) v = 0.f;
                    dV[idx] = v;
                }
            }
    }
}

// ------------------------------------------------------------------------------------------
// dW_t[c][k] = sum_p V_t[p][c] dM_t[p][k], contraction over P split across gridDim.z CTAs.
// With one split the result (times the mask) goes straight to dW; otherwise each split writes
// its partial sum to scratch memory and conv_dw_reduce_kernel adds them in a fixed order.
// ------------------------------------------------------------------------------------------
template <int LAYOUT>
__global__ void __launch_bounds__(256) conv_dw_ffma_kernel(const float *__restrict__ V, const float *__restrict__ dY,
                                                             const float *__restrict__ mask, float *__restrict__ out, long long P,
                                                             int nH, int nW, int H, int W, int C, int K, int chunks_per_split,
                                                             int direct)
{
    __shared__ __align__(16) float Vs[4][kCh][kTN];   // [j][pp][cc]
    __shared__ __align__(16) float Ms[4][kCh][kTN];   // [j][pp][kk]
    const int tid = threadIdx.x;
    const int tc = tid & 15, tk = tid >> 4;
    const int ktiles = cdiv(K, kTN);
    const int c0 = (blockIdx.x / ktiles) * kTN;
    const int k0 = (blockIdx.x % ktiles) * kTN;
    const int i = blockIdx.y;
    const int split = blockIdx.z;

    float acc[4][4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[j][a][b] = 0.f;

    const long long pbeg = (long long)split * chunks_per_split * kCh;
    const long long pend = min(P, pbeg + (long long)chunks_per_split * kCh);
#pragma unroll 1
    for (long long pc = pbeg; pc < pend; pc += kCh) {
        __syncthreads();
#pragma unroll 1
        for (int e = tid; e < 4 * kCh * kTN; e += 256) {
            const int cc = e % kTN, pp = (e / kTN) % kCh, j = e / (kCh * kTN);
            float v = 0.f;
            if (pc + pp < pend && c0 + cc < C) v = __ldg(V + ((long long)(4 * i + j) * P + pc + pp) * C + c0 + cc);
            Vs[j][pp][cc] = v;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = tid + 256 * r;
            const int kk = LAYOUT == WG2X2_NHWC ? (e % kTN) : (e / kCh);
            const int pp = LAYOUT == WG2X2_NHWC ? (e / kTN) : (e % kCh);
            float dm[4] = {0.f, 0.f, 0.f, 0.f};
            if (pc + pp < pend && k0 + kk < K) {
                float g[2][2];
                load_dy_block<LAYOUT>(dY, pc + pp, k0 + kk, nH, nW, H, W, K, g);
                a_g_at_row(i, g[0][0], g[0][1], g[1][0], g[1][1], dm);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) Ms[j][pp][kk] = dm[j];
        }
        __syncthreads();
#pragma unroll
        for (int pp = 0; pp < kCh; ++pp) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 a = *reinterpret_cast<const float4 *>(&Vs[j][pp][4 * tc]);
                const float4 w = *reinterpret_cast<const float4 *>(&Ms[j][pp][4 * tk]);
                const float av[4] = {a.x, a.y, a.z, a.w};
                const float wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int ci = 0; ci < 4; ++ci)
#pragma unroll
                    for (int ki = 0; ki < 4; ++ki) acc[j][ci][ki] = fmaf(av[ci], wv[ki], acc[j][ci][ki]);
            }
        }
    }
    float *dst = direct ? out : out + (long long)split * 16 * C * K;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
            const int c = c0 + 4 * tc + ci;
            if (c >= C) continue;
#pragma unroll
            for (int ki = 0; ki < 4; ++ki) {
                const int k = k0 + 4 * tk + ki;
                if (k >= K) continue;
                const long long idx = ((long long)(4 * i + j) * C + c) * K + k;
                float v = acc[j][ci][ki];
                if (direct && mask) v *= __ldg(mask + idx);
                dst[idx] = v;
            }
        }
}

__global__ void __launch_bounds__(256) conv_dw_reduce_kernel(const float *__restrict__ partial, const float *__restrict__ mask,
                                                               float *__restrict__ dW, long long n, int splits)
{
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int sp = 0; sp < splits; ++sp) s += partial[(long long)sp * n + idx];
        if (mask) s *= __ldg(mask + idx);
        dW[idx] = s;
    }
}

void dw_reduce_launch(const float *partial, const float *mask, float *dW, long long n, int splits, cudaStream_t st)
{
    const int blocks = (int)min((long long)kNumSMs * 8, cdivll(n, 256));
    conv_dw_reduce_kernel<<<blocks, 256, 0, st>>>(partial, mask, dW, n, splits);
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int conv_fwd_ffma(const float *V, const float *Wt, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW,
                  int layout, cudaStream_t st)
{
    const long long P = (long long)B * nH * nW;
    const long long gx = cdivll(P, kTP);
    if (gx > 0x7fffffffLL || cdiv(K, kTN) > 65535) return WG2X2_ERR_UNSUPPORTED;
    dim3 grid((unsigned)gx, cdiv(K, kTN));
    const bool vec = (C % 4 == 0) && (K % 4 == 0) && aligned16(V) && aligned16(Wt) && aligned16(Y);
    if (layout == WG2X2_NHWC) {
        if (vec) conv_fwd_ffma_kernel<true, WG2X2_NHWC><<<grid, 256, 0, st>>>(V, Wt, Y, P, nH, nW, C, K, outH, outW);
        else     conv_fwd_ffma_kernel<false, WG2X2_NHWC><<<grid, 256, 0, st>>>(V, Wt, Y, P, nH, nW, C, K, outH, outW);
    } else {
        if (vec) conv_fwd_ffma_kernel<true, WG2X2_NCHW><<<grid, 256, 0, st>>>(V, Wt, Y, P, nH, nW, C, K, outH, outW);
        else     conv_fwd_ffma_kernel<false, WG2X2_NCHW><<<grid, 256, 0, st>>>(V, Wt, Y, P, nH, nW, C, K, outH, outW);
    }
    return launch_status();
}

int conv_dv_ffma(const float *V, const float *Wt, const float *dY, float *dV, int B, int H, int W, int C, int K, int layout,
                 int relu, cudaStream_t st)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const long long P = (long long)B * nH * nW;
    const long long gx = cdivll(P, kTP);
    if (gx > 0x7fffffffLL || cdiv(C, kTN) > 65535) return WG2X2_ERR_UNSUPPORTED;
    dim3 grid((unsigned)gx, cdiv(C, kTN));
    if (layout == WG2X2_NHWC) conv_dv_ffma_kernel<WG2X2_NHWC><<<grid, 256, 0, st>>>(V, Wt, dY, dV, P, nH, nW, H, W, C, K, relu);
    else                      conv_dv_ffma_kernel<WG2X2_NCHW><<<grid, 256, 0, st>>>(V, Wt, dY, dV, P, nH, nW, H, W, C, K, relu);
    return launch_status();
}

// Number of P-splits of the dW kernel: enough CTAs for about two waves over the SMs.
int conv_dw_splits(long long P, int C, int K)
{
    const long long tiles = (long long)cdiv(C, kTN) * cdiv(K, kTN) * 4;
    const long long chunks = cdivll(P, kCh);
    long long s = cdivll(2 * kNumSMs, tiles);
    if (s > chunks) s = chunks;
    if (s > 1024) s = 1024;
    if (s < 1) s = 1;
    // every split must own at least one chunk
    const long long cps = cdivll(chunks, s);
    return (int)cdivll(chunks, cps);
}

size_t conv_dw_scratch_bytes(long long P, int C, int K)
{
    const int s = conv_dw_splits(P, C, K);
    return s > 1 ? (size_t)s * 16 * C * K * sizeof(float) : 0;
}

int conv_dw_ffma(const float *V, const float *dY, const float *mask, float *dW, int B, int H, int W, int C, int K, int layout,
                 float *scratch, int splits, cudaStream_t st)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const long long P = (long long)B * nH * nW;
    const long long chunks = cdivll(P, kCh);
    const int cps = (int)cdivll(chunks, splits);
    const long long gx = (long long)cdiv(C, kTN) * cdiv(K, kTN);
    if (gx > 0x7fffffffLL || splits > 65535) return WG2X2_ERR_UNSUPPORTED;
    dim3 grid((unsigned)gx, 4, splits);
    const int direct = splits == 1;
    float *out = direct ? dW : scratch;
    if (layout == WG2X2_NHWC) conv_dw_ffma_kernel<WG2X2_NHWC><<<grid, 256, 0, st>>>(V, dY, mask, out, P, nH, nW, H, W, C, K, cps, direct);
    else                      conv_dw_ffma_kernel<WG2X2_NCHW><<<grid, 256, 0, st>>>(V, dY, mask, out, P, nH, nW, H, W, C, K, cps, direct);
    if (launch_status() != WG2X2_OK) return WG2X2_ERR_LAUNCH;
    if (!direct) {
        const long long n = (long long)16 * C * K;
        const int blocks = (int)min((long long)kNumSMs * 8, cdivll(n, 256));
        conv_dw_reduce_kernel<<<blocks, 256, 0, st>>>(scratch, mask, dW, n, splits);
    }
    return launch_status();
}

}  // namespace wg
