// Input transform (+ Winograd-domain ReLU) and its gradient.  HBM-bound kernels:
//   forward  : reads |X| once from HBM (the 4x overlap between neighbouring tiles is served
//              by L1/L2 or by the shared-memory stage), writes 16 planes of V = 4|X|
//   backward : reads dV (and V when the ReLU mask is asked for), writes dX; a gather, so it
//              is deterministic and needs neither atomics nor scratch memory.
#include "wg_common.cuh"

namespace wg {

template <int VEC> struct Vec;
template <> struct Vec<4> { using type = float4; };
template <> struct Vec<1> { using type = float; };

__device__ __forceinline__ float4 ldg(const float4 *p) { return __ldg(p); }
__device__ __forceinline__ float ldg(const float *p) { return __ldg(p); }
__device__ __forceinline__ float4 zero_of(float4) { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float zero_of(float) { return 0.f; }
__device__ __forceinline__ float4 fma_of(float4 a, float4 s, float4 b) { return make_float4(fmaf(a.x, s.x, b.x), fmaf(a.y, s.y, b.y), fmaf(a.z, s.z, b.z), fmaf(a.w, s.w, b.w)); }
__device__ __forceinline__ float fma_of(float a, float s, float b) { return fmaf(a, s, b); }
__device__ __forceinline__ float4 relu_of(float4 a) { return make_float4(fmaxf(a.x, 0.f), fmaxf(a.y, 0.f), fmaxf(a.z, 0.f), fmaxf(a.w, 0.f)); }
__device__ __forceinline__ float relu_of(float a) { return fmaxf(a, 0.f); }
// the components of a value to p[0], p[pitch], ... (by name: indexing through a pointer would put the value on the stack)
__device__ __forceinline__ void put_lanes(float *p, int pitch, float4 v) { p[0] = v.x; p[pitch] = v.y; p[2 * pitch] = v.z; p[3 * pitch] = v.w; }
__device__ __forceinline__ void put_lanes(float *p, int, float v) { p[0] = v; }
__device__ __forceinline__ float4 keep_where_pos(float4 g, float4 m) { return make_float4(m.x > 0.f ? g.x : 0.f, m.y > 0.f ? g.y : 0.f, m.z > 0.f ? g.z : 0.f, m.w > 0.f ? g.w : 0.f); }
__device__ __forceinline__ float keep_where_pos(float g, float m) { return m > 0.f ? g : 0.f; }

// ------------------------------------------------------------------------------------------
// Forward, NHWC.  One thread = one tile x VEC channels; consecutive threads walk the channel
// axis first, so each of the 16 plane stores of a warp is one contiguous run.
// ------------------------------------------------------------------------------------------
template <int VEC, bool AFFINE>
__global__ void __launch_bounds__(256) imtrans_fwd_nhwc_kernel(const float *__restrict__ X, float *__restrict__ V,
                                                                 int B, int H, int W, int C, int nH, int nW, int relu,
                                                                 const float *__restrict__ scale, const float *__restrict__ shift)
{
    using T = typename Vec<VEC>::type;
    const int CV = C / VEC;
    const long long total = (long long)B * nH * nW * CV;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int cv = (int)(idx % CV);
    const long long p = idx / CV;
    const int tw = (int)(p % nW);
    const int th = (int)((p / nW) % nH);
    const int b = (int)(p / ((long long)nW * nH));

    const T *Xv = reinterpret_cast<const T *>(X);
    // optional per-channel affine map of the pixels (an inference-form BatchNorm in front of the
    // transform); the zero padding stays zero
    T sc = zero_of(T()), sh = zero_of(T());
    if (AFFINE) { sc = ldg(reinterpret_cast<const T *>(scale) + cv); sh = ldg(reinterpret_cast<const T *>(shift) + cv); }
    T d[4][4];
#pragma unroll
    for (int y = 0; y < 4; ++y) {
        const int fy = 2 * th - 1 + y;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int fx = 2 * tw - 1 + x;
            const bool in = (fy >= 0) && (fy < H) && (fx >= 0) && (fx < W);
            T v = in ? ldg(Xv + (((long long)b * H + fy) * W + fx) * CV + cv) : zero_of(T());
            if (AFFINE && in) v = fma_of(v, sc, sh);
            d[y][x] = v;
        }
    }
    T v[4][4];
    bt_d_b(d, v);
    T *Vv = reinterpret_cast<T *>(V);
    const long long plane = (long long)B * nH * nW * CV;
    const long long off = p * CV + cv;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            Vv[(long long)(4 * i + j) * plane + off] = relu ? relu_of(v[i][j]) : v[i][j];
}

// ------------------------------------------------------------------------------------------
// Forward, NCHW.  The image axis W is contiguous and tiles overlap along it, so a CTA stages
// the 4 input rows of one tile row, for CCH channels and TSEG tiles, in shared memory
// (coalesced along W), then computes with the channel index fastest across a warp so that
// the plane stores are contiguous along C.
// ------------------------------------------------------------------------------------------
constexpr int kCCH = 32;                       // channels per CTA
constexpr int kTSEG = 32;                      // tiles along W per CTA
constexpr int kRowPitch = 2 * kTSEG + 2;       // 66 pixels feed 32 tiles
constexpr int kChanPitch = 4 * kRowPitch + 1;  // odd, so 32 channels hit 32 different banks

__global__ void __launch_bounds__(256) imtrans_fwd_nchw_kernel(const float *__restrict__ X, float *__restrict__ V,
                                                                 int B, int H, int W, int C, int nH, int nW, int relu,
                                                                 const float *__restrict__ scale, const float *__restrict__ shift)
{
    __shared__ float S[kCCH * kChanPitch];
    const int nseg = cdiv(nW, kTSEG);
    int bx = blockIdx.x;
    const int seg = bx % nseg; bx /= nseg;
    const int th = bx % nH;
    const int b = bx / nH;
    const int c0 = blockIdx.y * kCCH;
    const int tw0 = seg * kTSEG;
    const int tid = threadIdx.x;

    for (int idx = tid; idx < kCCH * 4 * kRowPitch; idx += 256) {
        const int x = idx % kRowPitch;
        const int y = (idx / kRowPitch) & 3;
        const int c = idx / (4 * kRowPitch);
        const int gx = 2 * tw0 - 1 + x, gy = 2 * th - 1 + y;
        float val = 0.f;
        if (c0 + c < C && gx >= 0 && gx < W && gy >= 0 && gy < H) {
            val = __ldg(X + (((long long)b * C + c0 + c) * H + gy) * W + gx);
            if (scale) val = fmaf(val, __ldg(scale + c0 + c), __ldg(shift + c0 + c));
        }
        S[c * kChanPitch + y * kRowPitch + x] = val;
    }
    __syncthreads();

    const int c = tid & 31;
    const long long plane = (long long)B * nH * nW * C;
#pragma unroll 1
    for (int it = 0; it < kTSEG / 8; ++it) {
        const int twl = (tid >> 5) + 8 * it;
        const int tw = tw0 + twl;
        if (tw >= nW || c0 + c >= C) continue;
        float d[4][4], v[4][4];
#pragma unroll
        for (int y = 0; y < 4; ++y)
#pragma unroll
            for (int x = 0; x < 4; ++x) d[y][x] = S[c * kChanPitch + y * kRowPitch + 2 * twl + x];
        bt_d_b(d, v);
        const long long off = (((long long)b * nH + th) * nW + tw) * C + c0 + c;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                V[(long long)(4 * i + j) * plane + off] = relu ? fmaxf(v[i][j], 0.f) : v[i][j];
    }
}

// ------------------------------------------------------------------------------------------
// Forward, NCHW, image rows up to 128 pixels (every Winograd layer of a ResNet).  A CTA owns one
// image, 32 channels and a band of R tile rows.  For one channel the 2R+2 input rows of the band
// are one contiguous run of memory, so the fill is a plain coalesced copy into shared memory
// (one run per channel, odd pitch between channels); then each warp walks tiles with lane =
// channel, which makes the shared-memory reads conflict-free and every plane store one
// contiguous 128-byte run along C.  Borders and padding are predicates on warp-uniform
// coordinates.  Rows are re-read (2R+2)/2R times, from L2.
// ------------------------------------------------------------------------------------------
constexpr int kBandFloats = 384;   // at most this many input floats per channel in shared memory

template <bool AFFINE>
__global__ void __launch_bounds__(256) imtrans_fwd_nchw_band_kernel(const float *__restrict__ X, float *__restrict__ V,
                                                                      int B, int H, int W, int C, int nH, int nW, int relu,
                                                                      int R, int nbands, int pitch,
                                                                      const float *__restrict__ scale, const float *__restrict__ shift)
{
    extern __shared__ float S[];   // [32 channels][pitch]
    const int band = blockIdx.x % nbands;
    const int b = blockIdx.x / nbands;
    const int c0 = blockIdx.y * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int th0 = band * R;
    const int rows_tile = min(R, nH - th0);
    const int gy0 = 2 * th0 - 1;                                  // first input row of the band (may be -1)
    const int lo = max(gy0, 0), hi = min(gy0 + 2 * rows_tile + 2, H);
    const int nfill = (hi - lo) * W;

    for (int cc = warp; cc < 32; cc += 8) {
        if (c0 + cc >= C) break;
        const float *src = X + (((long long)b * C + c0 + cc) * H + lo) * W;
        float *dst = S + cc * pitch + (lo - gy0) * W;
        for (int i = lane; i < nfill; i += 32) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    const long long plane = (long long)B * nH * nW * C;
    const bool c_ok = c0 + lane < C;
    const float *Sc = S + lane * pitch;
    const int ntiles = rows_tile * nW;
    const float sc = (AFFINE && c_ok) ? __ldg(scale + c0 + lane) : 1.f;
    const float sh = (AFFINE && c_ok) ? __ldg(shift + c0 + lane) : 0.f;
    for (int q = warp; q < ntiles; q += 8) {
        const int tr = q / nW, tw = q - tr * nW;
        float d[4][4], v[4][4];
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int gy = gy0 + 2 * tr + y;
            const bool row_ok = (gy >= 0) && (gy < H);
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int gx = 2 * tw - 1 + x;
                const bool in = row_ok && gx >= 0 && gx < W && c_ok;
                d[y][x] = in ? (AFFINE ? fmaf(Sc[(2 * tr + y) * W + gx], sc, sh) : Sc[(2 * tr + y) * W + gx]) : 0.f;
            }
        }
        bt_d_b(d, v);
        if (c_ok) {
            const long long off = (((long long)b * nH + th0 + tr) * nW + tw) * C + c0 + lane;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    V[(long long)(4 * i + j) * plane + off] = relu ? fmaxf(v[i][j], 0.f) : v[i][j];
        }
    }
}

// The same with four channels per lane: every plane store is 16 bytes per lane, 512 bytes per warp with LC = 32
// lanes along the channels (128 per CTA), 256 bytes with LC = 16 (64 per CTA, the two halves of a warp on two tiles
// at once).  Where the band is the whole image the CTA's channels are one contiguous run of X and are staged as such.
template <int LC, bool AFFINE>
__global__ void __launch_bounds__(256, 3) imtrans_fwd_nchw_vec_kernel(const float *__restrict__ X, float *__restrict__ V,
                                                                        int B, int H, int W, int C, int nH, int nW, int relu,
                                                                        int R, int nbands, int pitch,
                                                                        const float *__restrict__ scale, const float *__restrict__ shift)
{
    constexpr int CB = 4 * LC, QW = 32 / LC;
    extern __shared__ float S[];   // [CB channels][pitch]
    const int band = blockIdx.x % nbands;
    const int b = blockIdx.x / nbands;
    const int c0 = blockIdx.y * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lc = lane % LC, lq = lane / LC;
    const int th0 = band * R;
    const int rows_tile = min(R, nH - th0);
    const int gy0 = 2 * th0 - 1;                                  // first input row of the band (may be -1)
    const int lo = max(gy0, 0), hi = min(gy0 + 2 * rows_tile + 2, H);
    const int nfill = (hi - lo) * W;
    const int nch = min(CB, C - c0);
    if (nfill == H * W) {
        const float *src = X + ((long long)b * C + c0) * nfill;
        float *dst = S + (lo - gy0) * W;
        for (int k = threadIdx.x; k < nch * nfill; k += 256) {
            const int cc = k / nfill;
            dst[((cc & 3) * LC + (cc >> 2)) * pitch + (k - cc * nfill)] = __ldg(src + k);
        }
    } else {
        for (int cc = warp; cc < nch; cc += 8) {
            const float *src = X + (((long long)b * C + c0 + cc) * H + lo) * W;
            float *dst = S + ((cc & 3) * LC + (cc >> 2)) * pitch + (lo - gy0) * W;
            for (int i = lane; i < nfill; i += 32) dst[i] = __ldg(src + i);
        }
    }
    __syncthreads();
    if (c0 + 4 * lc >= C) return;

    const long long plane = (long long)B * nH * nW * C;
    // channel 4 * lc + ch sits in row ch * LC + lc: for a given ch the lanes read rows one odd pitch apart (no bank conflicts)
    const float *Sc = S + lc * pitch;
    float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
    if (AFFINE) {
        sc = __ldg(reinterpret_cast<const float4 *>(scale + c0) + lc);
        sh = __ldg(reinterpret_cast<const float4 *>(shift + c0) + lc);
    }
    const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, shv[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll 1
    for (int q = warp * QW + lq; q < rows_tile * nW; q += 8 * QW) {
        const int tr = q / nW, tw = q - tr * nW;
        float v[4][4][4];          // [channel][i][j]
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            float d[4][4];
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                const int gy = gy0 + 2 * tr + y;
                const bool row_ok = (gy >= 0) && (gy < H);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int gx = 2 * tw - 1 + x;
                    const bool in = row_ok && gx >= 0 && gx < W;
                    const float raw = in ? Sc[ch * LC * pitch + (2 * tr + y) * W + gx] : 0.f;
                    d[y][x] = in ? (AFFINE ? fmaf(raw, scv[ch], shv[ch]) : raw) : 0.f;
                }
            }
            bt_d_b(d, v[ch]);
        }
        const long long off = (((long long)b * nH + th0 + tr) * nW + tw) * C + c0 + 4 * lc;
        const float lo_v = relu ? 0.f : -__int_as_float(0x7f800000);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<float4 *>(V + (long long)(4 * i + j) * plane + off) =
                    make_float4(fmaxf(v[0][i][j], lo_v), fmaxf(v[1][i][j], lo_v), fmaxf(v[2][i][j], lo_v), fmaxf(v[3][i][j], lo_v));
    }
}

// ------------------------------------------------------------------------------------------
// Backward gather for one 2x2 output block (bh,bw) and VEC channels.
// dX[2bh+a][2bw+e] = sum over the 3x3 neighbourhood of tiles of G[y][x], y = a+1-2*dth,
// x = e+1-2*dtw, G = B g B^T, i.e. G[y][x] = sum_ij BT[i][y] BT[j][x] g[i][j].
// Everything below is unrolled with compile-time coefficients: the centre tile contributes
// its 16 values, the 4 edge neighbours 4 each, the 4 corner neighbours one each.
// ------------------------------------------------------------------------------------------
__host__ __device__ constexpr bool row_needed(int dt, int i)
{
    // dt=0 touches y in {1,2} (all i); dt=-1 touches y=3 (i=3 only); dt=+1 touches y=0 (i=0 only)
    return dt == 0 ? true : (dt < 0 ? i == 3 : i == 0);
}

template <typename T, bool MASK>
__device__ __forceinline__ void imtrans_bwd_block(const T *__restrict__ dV, const T *__restrict__ Vm, long long plane,
                                                  int b, int bh, int bw, int nH, int nW, int CV, int cv, T (&out)[2][2])
{
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) out[a][e] = zero_of(T());
#pragma unroll
    for (int dth = -1; dth <= 1; ++dth) {
        const int th = bh + dth;
        if (th < 0 || th >= nH) continue;
#pragma unroll
        for (int dtw = -1; dtw <= 1; ++dtw) {
            const int tw = bw + dtw;
            if (tw < 0 || tw >= nW) continue;
            const long long base = (((long long)b * nH + th) * nW + tw) * CV + cv;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (!row_needed(dth, i) || !row_needed(dtw, j)) continue;
                    T g = ldg(dV + (long long)(4 * i + j) * plane + base);
                    if (MASK) g = keep_where_pos(g, ldg(Vm + (long long)(4 * i + j) * plane + base));
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int y = a + 1 - 2 * dth, x = e + 1 - 2 * dtw;
                            if (y < 0 || y > 3 || x < 0 || x > 3) continue;
                            const int cf = bt_coef(i, y) * bt_coef(j, x);
                            if (cf > 0) out[a][e] = out[a][e] + g;
                            if (cf < 0) out[a][e] = out[a][e] - g;
                        }
                    }
                }
            }
        }
    }
}

template <int VEC, bool MASK>
__global__ void __launch_bounds__(256) imtrans_bwd_nhwc_kernel(const float *__restrict__ dV, const float *__restrict__ Vm,
                                                                 float *__restrict__ dX, int B, int H, int W, int C, int nH, int nW)
{
    using T = typename Vec<VEC>::type;
    const int CV = C / VEC;
    const long long total = (long long)B * nH * nW * CV;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int cv = (int)(idx % CV);
    const long long p = idx / CV;
    const int bw = (int)(p % nW);
    const int bh = (int)((p / nW) % nH);
    const int b = (int)(p / ((long long)nW * nH));
    T out[2][2];
    imtrans_bwd_block<T, MASK>(reinterpret_cast<const T *>(dV), reinterpret_cast<const T *>(Vm),
                               (long long)B * nH * nW * CV, b, bh, bw, nH, nW, CV, cv, out);
    T *dXv = reinterpret_cast<T *>(dX);
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int h = 2 * bh + a, w = 2 * bw + e;
            if (h < H && w < W) dXv[(((long long)b * H + h) * W + w) * CV + cv] = out[a][e];
        }
}

// NCHW: the same gather with the channel index fastest across a warp (coalesced dV reads), then a
// shared-memory turn so that dX rows are written contiguously along W.
template <bool MASK>
__global__ void __launch_bounds__(256) imtrans_bwd_nchw_kernel(const float *__restrict__ dV, const float *__restrict__ Vm,
                                                                 float *__restrict__ dX, int B, int H, int W, int C, int nH, int nW)
{
    constexpr int OP = 2 * kTSEG + 1;  // 65: odd pitch per (c,a) row
    __shared__ float O[kCCH * 2 * OP];
    const int nseg = cdiv(nW, kTSEG);
    int bx = blockIdx.x;
    const int seg = bx % nseg; bx /= nseg;
    const int bh = bx % nH;
    const int b = bx / nH;
    const int c0 = blockIdx.y * kCCH;
    const int bw0 = seg * kTSEG;
    const int tid = threadIdx.x;
    const int c = tid & 31;
    const long long plane = (long long)B * nH * nW * C;
#pragma unroll 1
    for (int it = 0; it < kTSEG / 8; ++it) {
        const int bwl = (tid >> 5) + 8 * it;
        const int bw = bw0 + bwl;
        float out[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        if (bw < nW && c0 + c < C)
            imtrans_bwd_block<float, MASK>(dV, Vm, plane, b, bh, bw, nH, nW, C, c0 + c, out);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e) O[(c * 2 + a) * OP + 2 * bwl + e] = out[a][e];
    }
    __syncthreads();
    for (int idx = tid; idx < kCCH * 2 * 2 * kTSEG; idx += 256) {
        const int x = idx % (2 * kTSEG);
        const int a = (idx / (2 * kTSEG)) & 1;
        const int cc = idx / (4 * kTSEG);
        const int h = 2 * bh + a, w = 2 * bw0 + x;
        if (c0 + cc < C && h < H && w < W)
            dX[(((long long)b * C + c0 + cc) * H + h) * W + w] = O[(cc * 2 + a) * OP + x];
    }
}

// NCHW, image rows up to 192 pixels: the same gather with lane = VEC consecutive channels over a band of R tile
// rows; the 2R x W output pixels of each channel collect in shared memory (odd pitch between channels) and
// leave as one contiguous run per channel -- or, where the band is the whole image, as one contiguous run for
// all the block's channels.  VEC = 4 reads dV (and the ReLU mask) with 16-byte loads: LC = 32 lanes along the
// channels (128 per block, 512 bytes per request) where such a band fits four blocks per SM, else LC = 16 (64
// channels per block, the two halves of a warp on two tiles at once).
template <int VEC, int LC, bool MASK>
__global__ void __launch_bounds__(256, 4) imtrans_bwd_nchw_band_kernel(const float *__restrict__ dV, const float *__restrict__ Vm,
                                                                         float *__restrict__ dX, int B, int H, int W, int C, int nH,
                                                                         int nW, int R, int nbands, int pitch)
{
    using T = typename Vec<VEC>::type;
    constexpr int CB = LC * VEC;             // channels per block
    constexpr int QW = 32 / LC;              // tiles a warp works on at once
    extern __shared__ float O[];             // [CB channels][pitch]
    // Block order.  One input stream: a one-dimensional grid with the channel blocks fastest, so that neighbouring
    // blocks read neighbouring segments of every dV row.  With the mask (32 streams of rows open at once) that
    // order measured slower than images fastest, which is the two-dimensional grid (66 vs 78 us on
    // 256 x 512 x 7 x 7; without the mask 50 vs 58 us the other way).
    int c0, bb;
    if (MASK) {
        c0 = blockIdx.y * CB;
        bb = blockIdx.x;
    } else {
        const int ncb = (C + CB - 1) / CB;
        c0 = (int)(blockIdx.x % ncb) * CB;
        bb = blockIdx.x / ncb;
    }
    const int band = bb % nbands;
    const int b = bb / nbands;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lc = lane % LC, lq = lane / LC;
    const int th0 = band * R;
    const int rows_blk = min(R, nH - th0);
    const int CV = C / VEC;
    const long long plane = (long long)B * nH * nW * CV;
    const bool c_ok = c0 + VEC * lc < C;
#pragma unroll 1
    for (int q = warp * QW + lq; q < rows_blk * nW; q += 8 * QW) {
        const int br = q / nW, bw = q - br * nW;
        T out[2][2];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e) out[a][e] = zero_of(T());
        if (c_ok)
            imtrans_bwd_block<T, MASK>(reinterpret_cast<const T *>(dV), reinterpret_cast<const T *>(Vm), plane, b, th0 + br, bw, nH,
                                       nW, CV, c0 / VEC + lc, out);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (2 * bw + e < W) {
                    float *o = O + VEC * lc * pitch + (2 * br + a) * W + 2 * bw + e;
                    put_lanes(o, pitch, out[a][e]);
                }
    }
    __syncthreads();
    const int lo = 2 * th0, hi = min(2 * th0 + 2 * rows_blk, H);
    const int n = (hi - lo) * W;
    const int nch = min(CB, C - c0);
    if (n == H * W) {
        // the block's channels are one run of nch * H * W floats
        float *dst = dX + ((long long)b * C + c0) * n;
        for (int k = threadIdx.x; k < nch * n; k += 256) {
            const int cc = k / n;
            dst[k] = O[cc * pitch + (k - cc * n)];
        }
    } else {
        for (int cc = warp; cc < nch; cc += 8) {
            float *dst = dX + (((long long)b * C + c0 + cc) * H + lo) * W;
            const float *src = O + cc * pitch;
            for (int i = lane; i < n; i += 32) dst[i] = src[i];
        }
    }
}


// NCHW, small images (a whole image of 128 or 64 channels fits shared memory): every value of dV is read from memory
// exactly once.  A block takes one image x CB channels; a warp takes one tile x 32 channels at a time (lane = channel:
// sixteen coalesced 128-byte loads), turns its sixteen gradients into the 4 x 4 window B g B^T and adds the window
// into the block's image in shared memory.  Windows of tiles two apart do not overlap, so the tiles are walked in four
// passes by the parity of (tile row, tile column) with a barrier between passes, and plain read-modify-writes suffice
// (no atomics: the result does not depend on the order of the warps).  The image is kept as [channel][pixel] with an
// odd pitch (lanes hit distinct banks) and leaves as one contiguous run: CB channels x H*W pixels are adjacent in dX.
template <bool MASK>
__global__ void __launch_bounds__(256) imtrans_bwd_nchw_image_kernel(const float *__restrict__ dV, const float *__restrict__ Vm,
                                                                       float *__restrict__ dX, int B, int H, int W, int C, int nH, int nW,
                                                                       int CB, int pitch)
{
    extern __shared__ float O[];                   // [CB][pitch]
    const int b = blockIdx.x, c0 = blockIdx.y * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HW = H * W;
    const int nch = min(CB, C - c0);
    const int ngr = (nch + 31) >> 5;               // groups of 32 channels
    const long long plane = (long long)B * nH * nW * C;
    for (int k = threadIdx.x; k < CB * pitch; k += 256) O[k] = 0.f;
    __syncthreads();
#pragma unroll 1
    for (int pc = 0; pc < 4; ++pc) {
        const int pr = pc >> 1, pq = pc & 1;
        const int ntr = (nH - pr + 1) >> 1, ntc = (nW - pq + 1) >> 1;
        const int ntiles = ntr * ntc;
        // (tile, channel group) pairs go round the eight warps; with 1, 2, 4 or 8 groups a warp keeps its group and
        // walks the tiles with a fixed stride, which keeps divisions out of the loop
        const bool fixed = (8 % ngr) == 0;
        const int step = fixed ? 8 / ngr : 8;
        int gr = fixed ? warp % ngr : 0, tt = fixed ? warp / ngr : warp;
        int tr = tt / ntc, tc = tt - tr * ntc;
        const int items = fixed ? ntiles : ntiles * ngr;
#pragma unroll 1
        for (; tt < items; tt += step) {
            int th, tw;
            if (fixed) {
                th = 2 * tr + pr; tw = 2 * tc + pq;
                tc += step;
                while (tc >= ntc) { tc -= ntc; ++tr; }
            } else {
                gr = tt % ngr;
                const int t2 = tt / ngr;
                th = 2 * (t2 / ntc) + pr; tw = 2 * (t2 % ntc) + pq;
            }
            const int cl = gr * 32 + lane;
            if (cl < nch) {
                const float *gp = dV + ((((long long)b * nH + th) * nW + tw) * C + c0 + cl);
                const float *vp = MASK ? Vm + ((((long long)b * nH + th) * nW + tw) * C + c0 + cl) : nullptr;
                float g[4][4];
#pragma unroll
                for (int t = 0; t < 16; ++t) g[t >> 2][t & 3] = __ldg(gp + (long long)t * plane);
                if (MASK) {
                    float v[16];
#pragma unroll
                    for (int t = 0; t < 16; ++t) v[t] = __ldg(vp + (long long)t * plane);
#pragma unroll
                    for (int t = 0; t < 16; ++t)
                        if (!(v[t] > 0.f)) g[t >> 2][t & 3] = 0.f;
                }
                // d = B g B^T, B[y][i] = Bt[i][y]: along one axis (u0..u3) -> (u0, u1 - u2 + u3, -u0 + u1 + u2, -u3)
                float r[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    r[0][j] = g[0][j];
                    r[1][j] = g[1][j] - g[2][j] + g[3][j];
                    r[2][j] = g[1][j] + g[2][j] - g[0][j];
                    r[3][j] = -g[3][j];
                }
                float *o = O + cl * pitch;
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int h = 2 * th - 1 + y;
                    if (h < 0 || h >= H) continue;
                    const float d0 = r[y][0], d1 = r[y][1] - r[y][2] + r[y][3], d2 = r[y][1] + r[y][2] - r[y][0], d3 = -r[y][3];
                    const int w0 = 2 * tw - 1;
                    float *row = o + h * W;
                    if (w0 >= 0) row[w0] += d0;
                    row[w0 + 1] += d1;
                    if (w0 + 2 < W) row[w0 + 2] += d2;
                    if (w0 + 3 < W) row[w0 + 3] += d3;
                }
            }
        }
        __syncthreads();
    }
    float *dst = dX + ((long long)b * C + c0) * HW;
    if (pitch == HW) {
        for (int k = threadIdx.x; k < nch * HW; k += 256) dst[k] = O[k];
    } else {   // a warp per channel: no division per element, and the channels' runs are adjacent in dX
        for (int c = warp; c < nch; c += 8) {
            const float *src = O + c * pitch;
            float *d = dst + c * HW;
            for (int i = lane; i < HW; i += 32) d[i] = src[i];
        }
    }
}

// The same with two channels per lane (8-byte loads, a warp covers a tile x 64 channels): half the instructions per byte,
// which is what this kernel is short of.  The image is kept as [pixel][channel] (channels innermost, so that the lanes'
// 8-byte read-modify-writes are conflict-free) with a pitch of CB + 2 floats, and leaves per channel through strided
// reads (two-way bank conflicts on the smaller side of the traffic).  Needs an even C and 8-byte aligned tensors.
__device__ __forceinline__ float2 f2add(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 f2sub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ float2 f2neg(float2 a) { return make_float2(-a.x, -a.y); }

template <bool MASK>
__global__ void __launch_bounds__(256, 4) imtrans_bwd_nchw_image2_kernel(const float *__restrict__ dV, const float *__restrict__ Vm,
                                                                           float *__restrict__ dX, int B, int H, int W, int C, int nH,
                                                                           int nW, int CB)
{
    extern __shared__ __align__(16) float O[];     // [H*W][CB + 2]
    const int b = blockIdx.x, c0 = blockIdx.y * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HW = H * W, CBP = CB + 2;
    const int nch = min(CB, C - c0);
    const int ngr = (nch + 63) >> 6;               // groups of 64 channels
    const long long plane = (long long)B * nH * nW * C;
    for (int k = threadIdx.x; k < HW * CBP / 2; k += 256) reinterpret_cast<float2 *>(O)[k] = make_float2(0.f, 0.f);
    __syncthreads();
#pragma unroll 1
    for (int pc = 0; pc < 4; ++pc) {
        const int pr = pc >> 1, pq = pc & 1;
        const int ntr = (nH - pr + 1) >> 1, ntc = (nW - pq + 1) >> 1;
        const int items = ntr * ntc * ngr;
#pragma unroll 1
        for (int tt = warp; tt < items; tt += 8) {
            const int gr = tt % ngr, t2 = tt / ngr;
            const int th = 2 * (t2 / ntc) + pr, tw = 2 * (t2 % ntc) + pq;
            const int cl = gr * 64 + 2 * lane;
            if (cl < nch) {
                const long long base = (((long long)b * nH + th) * nW + tw) * C + c0 + cl;
                float2 g[4][4];
#pragma unroll
                for (int t = 0; t < 16; ++t) g[t >> 2][t & 3] = __ldg(reinterpret_cast<const float2 *>(dV + base + (long long)t * plane));
                if (MASK) {
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        const float2 v = __ldg(reinterpret_cast<const float2 *>(Vm + base + (long long)t * plane));
                        if (!(v.x > 0.f)) g[t >> 2][t & 3].x = 0.f;
                        if (!(v.y > 0.f)) g[t >> 2][t & 3].y = 0.f;
                    }
                }
                // d = B g B^T: along one axis (u0..u3) -> (u0, u1 - u2 + u3, -u0 + u1 + u2, -u3); rows in place
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 u1 = g[1][j], u2 = g[2][j];
                    g[1][j] = f2add(f2sub(u1, u2), g[3][j]);
                    g[2][j] = f2sub(f2add(u1, u2), g[0][j]);
                    g[3][j] = f2neg(g[3][j]);
                }
                float *o = O + cl;
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int h = 2 * th - 1 + y;
                    if (h < 0 || h >= H) continue;
                    const float2 d0 = g[y][0], d1 = f2add(f2sub(g[y][1], g[y][2]), g[y][3]), d2 = f2sub(f2add(g[y][1], g[y][2]), g[y][0]),
                                 d3 = f2neg(g[y][3]);
                    const int w0 = 2 * tw - 1;
                    float *row = o + (h * W + w0) * CBP;
                    if (w0 >= 0) { float2 *q = reinterpret_cast<float2 *>(row); *q = f2add(*q, d0); }
                    { float2 *q = reinterpret_cast<float2 *>(row + CBP); *q = f2add(*q, d1); }
                    if (w0 + 2 < W) { float2 *q = reinterpret_cast<float2 *>(row + 2 * CBP); *q = f2add(*q, d2); }
                    if (w0 + 3 < W) { float2 *q = reinterpret_cast<float2 *>(row + 3 * CBP); *q = f2add(*q, d3); }
                }
            }
        }
        __syncthreads();
    }
    // a warp per channel: its H*W pixels are one contiguous run of dX, and the channels' runs are adjacent
    float *dst = dX + ((long long)b * C + c0) * HW;
    for (int c = warp; c < nch; c += 8) {
        float *d = dst + c * HW;
        for (int i = lane; i < HW; i += 32) d[i] = O[i * CBP + c];
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int imtrans_fwd(const float *X, float *V, int B, int H, int W, int C, int layout, int relu, const float *scale, const float *shift,
                cudaStream_t st)
{
    if (!X || !V || B <= 0 || H <= 0 || W <= 0 || C <= 0) return WG2X2_ERR_BAD_ARG;
    if ((scale == nullptr) != (shift == nullptr)) return WG2X2_ERR_BAD_ARG;
    if (layout != WG2X2_NHWC && layout != WG2X2_NCHW) return WG2X2_ERR_BAD_ARG;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    if (layout == WG2X2_NHWC) {
        if ((C % 4 == 0) && aligned16(X) && aligned16(V) && (!scale || (aligned16(scale) && aligned16(shift)))) {
            const long long total = (long long)B * nH * nW * (C / 4);
            const unsigned g = (unsigned)cdivll(total, 256);
            if (scale) imtrans_fwd_nhwc_kernel<4, true><<<g, 256, 0, st>>>(X, V, B, H, W, C, nH, nW, relu, scale, shift);
            else       imtrans_fwd_nhwc_kernel<4, false><<<g, 256, 0, st>>>(X, V, B, H, W, C, nH, nW, relu, scale, shift);
        } else {
            const long long total = (long long)B * nH * nW * C;
            const unsigned g = (unsigned)cdivll(total, 256);
            if (scale) imtrans_fwd_nhwc_kernel<1, true><<<g, 256, 0, st>>>(X, V, B, H, W, C, nH, nW, relu, scale, shift);
            else       imtrans_fwd_nhwc_kernel<1, false><<<g, 256, 0, st>>>(X, V, B, H, W, C, nH, nW, relu, scale, shift);
        }
    } else {
        const long long gx = (long long)B * nH * cdiv(nW, kTSEG);
        if (gx > 0x7fffffffLL || cdiv(C, kCCH) > 65535) return WG2X2_ERR_UNSUPPORTED;
        dim3 grid((unsigned)gx, cdiv(C, kCCH));
        // Four channels per lane, 128 per CTA, where the whole image is one small band (7 x 7: 39.8 against 43.5 us on
        // 256 x 512 channels) and the CTAs still fill the GPU.  With several bands per image, or 64 channels per CTA
        // and a 14 x 14 image, the one-channel-per-lane kernel below measured faster (33 against 39-52 us).
        const int rows_all = 2 * nH + 2;
        const bool wide = (C % 4 == 0) && C >= 128 && aligned16(V) && (!scale || (aligned16(scale) && aligned16(shift))) &&
                          rows_all * W <= 96 && (long long)B * cdiv(C, 128) >= 4LL * kNumSMs;
        const bool vec = wide;
        if (vec) {
            const int cb = 128;
            const int R = nH, nbands = 1;
            const int pitch = ((2 * R + 2) * W) | 1;
            const int smem = cb * pitch * (int)sizeof(float);
            if ((long long)B * nbands > 0x7fffffffLL || cdiv(C, cb) > 65535) return WG2X2_ERR_UNSUPPORTED;
            const dim3 gb((unsigned)(B * nbands), cdiv(C, cb));
            auto launch = [&](auto kernel) -> bool {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return false;
                kernel<<<gb, 256, smem, st>>>(X, V, B, H, W, C, nH, nW, relu, R, nbands, pitch, scale, shift);
                return true;
            };
            const bool launched = scale ? launch(imtrans_fwd_nchw_vec_kernel<32, true>) : launch(imtrans_fwd_nchw_vec_kernel<32, false>);
            if (!launched) return WG2X2_ERR_LAUNCH;
        } else if (W <= 128) {
            int R = (kBandFloats / W - 2) / 2;
            if (R < 1) R = 1;
            if (R > nH) R = nH;
            // a small batch: lower bands, so that the grid still gives every SM a few blocks
            while (R > 1 && (long long)B * cdiv(nH, R) * cdiv(C, 32) < 3LL * kNumSMs) --R;
            const int nbands = cdiv(nH, R);
            R = cdiv(nH, nbands);
            const int pitch = ((2 * R + 2) * W) | 1;
            const int smem = 32 * pitch * (int)sizeof(float);
            const long long gxb = (long long)B * nbands;
            if (gxb > 0x7fffffffLL) return WG2X2_ERR_UNSUPPORTED;
            const dim3 gb((unsigned)gxb, cdiv(C, 32));
            if (scale) {
                if (cudaFuncSetAttribute(imtrans_fwd_nchw_band_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                    return WG2X2_ERR_LAUNCH;
                imtrans_fwd_nchw_band_kernel<true><<<gb, 256, smem, st>>>(X, V, B, H, W, C, nH, nW, relu, R, nbands, pitch, scale, shift);
            } else {
                if (cudaFuncSetAttribute(imtrans_fwd_nchw_band_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                    return WG2X2_ERR_LAUNCH;
                imtrans_fwd_nchw_band_kernel<false><<<gb, 256, smem, st>>>(X, V, B, H, W, C, nH, nW, relu, R, nbands, pitch, scale, shift);
            }
        } else {
            imtrans_fwd_nchw_kernel<<<grid, 256, 0, st>>>(X, V, B, H, W, C, nH, nW, relu, scale, shift);
        }
    }
    return launch_status();
}

int imtrans_bwd(const float *dV, const float *Vm, float *dX, int B, int H, int W, int C, int layout, cudaStream_t st)
{
    if (!dV || !dX || B <= 0 || H <= 0 || W <= 0 || C <= 0) return WG2X2_ERR_BAD_ARG;
    if (layout != WG2X2_NHWC && layout != WG2X2_NCHW) return WG2X2_ERR_BAD_ARG;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    if (layout == WG2X2_NHWC) {
        const bool vec = (C % 4 == 0) && aligned16(dV) && aligned16(dX) && (!Vm || aligned16(Vm));
        const long long total = (long long)B * nH * nW * (vec ? C / 4 : C);
        const unsigned g = (unsigned)cdivll(total, 256);
        if (vec) {
            if (Vm) imtrans_bwd_nhwc_kernel<4, true><<<g, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
            else    imtrans_bwd_nhwc_kernel<4, false><<<g, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
        } else {
            if (Vm) imtrans_bwd_nhwc_kernel<1, true><<<g, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
            else    imtrans_bwd_nhwc_kernel<1, false><<<g, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
        }
    } else {
        // small images: one block per image and channel block, every value of dV read once
        const int HW = H * W;
        if (HW <= 200 && (long long)B * cdiv(C, HW <= 64 ? 128 : 64) >= 2LL * kNumSMs && B <= 0x7fffffff) {
            const int CB = HW <= 64 ? 128 : 64;
            const auto aligned8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7u) == 0; };
            if ((C & 1) == 0 && aligned8(dV) && (!Vm || aligned8(Vm)) && cdiv(C, CB) <= 65535) {      // two channels per lane
                const int smem2 = HW * (CB + 2) * (int)sizeof(float);
                const dim3 grid2((unsigned)B, cdiv(C, CB));
                if (Vm) {
                    if (cudaFuncSetAttribute(imtrans_bwd_nchw_image2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) != cudaSuccess)
                        return WG2X2_ERR_LAUNCH;
                    imtrans_bwd_nchw_image2_kernel<true><<<grid2, 256, smem2, st>>>(dV, Vm, dX, B, H, W, C, nH, nW, CB);
                } else {
                    if (cudaFuncSetAttribute(imtrans_bwd_nchw_image2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) != cudaSuccess)
                        return WG2X2_ERR_LAUNCH;
                    imtrans_bwd_nchw_image2_kernel<false><<<grid2, 256, smem2, st>>>(dV, Vm, dX, B, H, W, C, nH, nW, CB);
                }
                return launch_status();
            }
            const int pitch = HW | 1;
            const int smem = CB * pitch * (int)sizeof(float);
            if (cdiv(C, CB) <= 65535) {
                const dim3 grid((unsigned)B, cdiv(C, CB));
                if (Vm) {
                    if (cudaFuncSetAttribute(imtrans_bwd_nchw_image_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                        return WG2X2_ERR_LAUNCH;
                    imtrans_bwd_nchw_image_kernel<true><<<grid, 256, smem, st>>>(dV, Vm, dX, B, H, W, C, nH, nW, CB, pitch);
                } else {
                    if (cudaFuncSetAttribute(imtrans_bwd_nchw_image_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
                        return WG2X2_ERR_LAUNCH;
                    imtrans_bwd_nchw_image_kernel<false><<<grid, 256, smem, st>>>(dV, Vm, dX, B, H, W, C, nH, nW, CB, pitch);
                }
                return launch_status();
            }
        }
        if (W <= 192) {
            // four channels per lane (16-byte loads) where the channels allow it and a band of 128 channels stays small
            // four channels per lane (16-byte loads) where the channels allow it; 128 channels per block where a band of
            // them stays below 50 KB (four blocks per SM), else 64
            // -- and where that still leaves four CTAs for every SM (a small batch keeps the narrower blocks)
            auto ctas = [&](int cbk, int band_floats) { return (long long)B * cdiv(nH, max(1, min(nH, band_floats / (2 * W)))) * cdiv(C, cbk); };
            const long long fill = 4LL * kNumSMs;
            const bool vec_ok = (C % 4 == 0) && C >= 64 && aligned16(dV) && (!Vm || aligned16(Vm)) && 2 * W <= kBandFloats / 2;
            const bool wide = vec_ok && C >= 128 && 2 * W <= kBandFloats / 4 && ctas(128, kBandFloats / 4) >= fill;
            const bool vec = wide || (vec_ok && ctas(64, kBandFloats / 2) >= fill);
            const int cb = wide ? 128 : (vec ? 64 : 32);
            int R = (wide ? kBandFloats / 4 : (vec ? kBandFloats / 2 : kBandFloats)) / (2 * W);
            if (R < 1) R = 1;
            if (R > nH) R = nH;
            const int nbands = cdiv(nH, R);
            R = cdiv(nH, nbands);                              // bands of even height
            const int pitch = (2 * R * W) | 1;
            const int smem = cb * pitch * (int)sizeof(float);
            if ((long long)B * nbands * cdiv(C, cb) > 0x7fffffffLL || cdiv(C, cb) > 65535) return WG2X2_ERR_UNSUPPORTED;
            const dim3 grid = Vm ? dim3((unsigned)(B * nbands), cdiv(C, cb)) : dim3((unsigned)(B * nbands * cdiv(C, cb)));
            auto launch = [&](auto kernel) -> bool {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return false;
                kernel<<<grid, 256, smem, st>>>(dV, Vm, dX, B, H, W, C, nH, nW, R, nbands, pitch);
                return true;
            };
            const bool launched =
                wide ? (Vm ? launch(imtrans_bwd_nchw_band_kernel<4, 32, true>) : launch(imtrans_bwd_nchw_band_kernel<4, 32, false>))
                : vec ? (Vm ? launch(imtrans_bwd_nchw_band_kernel<4, 16, true>) : launch(imtrans_bwd_nchw_band_kernel<4, 16, false>))
                      : (Vm ? launch(imtrans_bwd_nchw_band_kernel<1, 32, true>) : launch(imtrans_bwd_nchw_band_kernel<1, 32, false>));
            if (!launched) return WG2X2_ERR_LAUNCH;
            return launch_status();
        }
        const long long gx = (long long)B * nH * cdiv(nW, kTSEG);
        if (gx > 0x7fffffffLL || cdiv(C, kCCH) > 65535) return WG2X2_ERR_UNSUPPORTED;
        dim3 grid((unsigned)gx, cdiv(C, kCCH));
        if (Vm) imtrans_bwd_nchw_kernel<true><<<grid, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
        else    imtrans_bwd_nchw_kernel<false><<<grid, 256, 0, st>>>(dV, Vm, dX, B, H, W, C, nH, nW);
    }
    return launch_status();
}

}  // namespace wg
