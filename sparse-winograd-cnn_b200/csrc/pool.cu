// 3x3 / stride 2 max-pooling with TensorFlow's SAME padding on NCHW tensors, the down-sampling step between the
// stages of the reference's ResNet-18-var graph (MaxPooling('pool*', l, 3, stride=2, padding='SAME'),
// ResNet-18-var/imagenet-resnet-transWino-prune.py:115,141,166,191).  HBM-bound: every input element is read once
// from memory (the overlap of neighbouring windows is served by registers and L1), every output written once; an
// optional second output holds relu(pooled), which the next stage's shortcut branch starts from, so that it costs
// no pass of its own; with a per-channel scale and shift it is relu(scale * pooled + shift), the BNReLU the first
// stage's shortcut starts from (:126-127).
//
// SAME padding: the output has ceil(H/2) x ceil(W/2) pixels; for an even size the window of output i covers input
// 2i .. 2i+2 (one row/column of padding at the far end only), for an odd size 2i-1 .. 2i+1.  Padding never wins the
// maximum (it counts as -inf).
#include "wg_common.cuh"

namespace wg {

// Four consecutive outputs of a row per thread: input columns 8t .. 8t+8 of three rows = two 16-byte loads and one
// scalar per row.  Needs an even W that is a multiple of 8 and 16-byte aligned tensors.
template <bool RELU_OUT>
__global__ void __launch_bounds__(256) maxpool_vec_kernel(const float *__restrict__ X, float *__restrict__ Y, float *__restrict__ Yr,
                                                            const float *__restrict__ rs, const float *__restrict__ rb, int C,
                                                            long long planes, int H, int W, int OH, int OW, int ph)
{
    const int OW4 = OW >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = planes * OH * OW4;
    if (idx >= total) return;
    const int t = (int)(idx % OW4);
    const int oh = (int)((idx / OW4) % OH);
    const long long pl = idx / ((long long)OW4 * OH);
    const float *xp = X + pl * H * W;
    const float ninf = -__int_as_float(0x7f800000);
    float m[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) m[k] = ninf;
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
        const int h = 2 * oh - ph + dy;
        if (h < 0 || h >= H) continue;
        const float *row = xp + (long long)h * W + 8 * t;
        const float4 a = __ldg(reinterpret_cast<const float4 *>(row));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(row) + 1);
        const float c = (8 * t + 8 < W) ? __ldg(row + 8) : ninf;
        m[0] = fmaxf(m[0], a.x); m[1] = fmaxf(m[1], a.y); m[2] = fmaxf(m[2], a.z); m[3] = fmaxf(m[3], a.w);
        m[4] = fmaxf(m[4], b.x); m[5] = fmaxf(m[5], b.y); m[6] = fmaxf(m[6], b.z); m[7] = fmaxf(m[7], b.w);
        m[8] = fmaxf(m[8], c);
    }
    float4 o;
    o.x = fmaxf(fmaxf(m[0], m[1]), m[2]);
    o.y = fmaxf(fmaxf(m[2], m[3]), m[4]);
    o.z = fmaxf(fmaxf(m[4], m[5]), m[6]);
    o.w = fmaxf(fmaxf(m[6], m[7]), m[8]);
    const long long off = (pl * OH + oh) * OW + 4 * t;
    *reinterpret_cast<float4 *>(Y + off) = o;
    if (RELU_OUT) {
        const float sc = rs ? __ldg(rs + (int)(pl % C)) : 1.f, sh = rs ? __ldg(rb + (int)(pl % C)) : 0.f;
        *reinterpret_cast<float4 *>(Yr + off) = make_float4(fmaxf(fmaf(o.x, sc, sh), 0.f), fmaxf(fmaf(o.y, sc, sh), 0.f),
                                                            fmaxf(fmaf(o.z, sc, sh), 0.f), fmaxf(fmaf(o.w, sc, sh), 0.f));
    }
}

// Two consecutive outputs of a row per thread, for widths that are multiples of 4 but not of 8 (28 -> 14): input columns
// 4t .. 4t+4 of three rows = one 16-byte load and one scalar per row; the output pair is one 8-byte store.
template <bool RELU_OUT>
__global__ void __launch_bounds__(256) maxpool_vec2_kernel(const float *__restrict__ X, float *__restrict__ Y, float *__restrict__ Yr,
                                                             const float *__restrict__ rs, const float *__restrict__ rb, int C,
                                                             long long planes, int H, int W, int OH, int OW, int ph)
{
    const int OW2 = OW >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= planes * OH * OW2) return;
    const int t = (int)(idx % OW2);
    const int oh = (int)((idx / OW2) % OH);
    const long long pl = idx / ((long long)OW2 * OH);
    const float *xp = X + pl * H * W;
    const float ninf = -__int_as_float(0x7f800000);
    float m[5] = {ninf, ninf, ninf, ninf, ninf};
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
        const int h = 2 * oh - ph + dy;
        if (h < 0 || h >= H) continue;
        const float *row = xp + (long long)h * W + 4 * t;
        const float4 a = __ldg(reinterpret_cast<const float4 *>(row));
        const float c = (4 * t + 4 < W) ? __ldg(row + 4) : ninf;
        m[0] = fmaxf(m[0], a.x); m[1] = fmaxf(m[1], a.y); m[2] = fmaxf(m[2], a.z); m[3] = fmaxf(m[3], a.w);
        m[4] = fmaxf(m[4], c);
    }
    const float2 o = make_float2(fmaxf(fmaxf(m[0], m[1]), m[2]), fmaxf(fmaxf(m[2], m[3]), m[4]));
    const long long off = (pl * OH + oh) * OW + 2 * t;
    *reinterpret_cast<float2 *>(Y + off) = o;
    if (RELU_OUT) {
        const float sc = rs ? __ldg(rs + (int)(pl % C)) : 1.f, sh = rs ? __ldg(rb + (int)(pl % C)) : 0.f;
        *reinterpret_cast<float2 *>(Yr + off) = make_float2(fmaxf(fmaf(o.x, sc, sh), 0.f), fmaxf(fmaf(o.y, sc, sh), 0.f));
    }
}

// Any size: one output per thread.
template <bool RELU_OUT>
__global__ void __launch_bounds__(256) maxpool_any_kernel(const float *__restrict__ X, float *__restrict__ Y, float *__restrict__ Yr,
                                                            const float *__restrict__ rs, const float *__restrict__ rb, int C,
                                                            long long planes, int H, int W, int OH, int OW, int ph, int pw)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= planes * OH * OW) return;
    const int ow = (int)(idx % OW);
    const int oh = (int)((idx / OW) % OH);
    const long long pl = idx / ((long long)OW * OH);
    const float *xp = X + pl * H * W;
    float m = -__int_as_float(0x7f800000);
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
        const int h = 2 * oh - ph + dy;
        if (h < 0 || h >= H) continue;
#pragma unroll
        for (int dx = 0; dx < 3; ++dx) {
            const int w = 2 * ow - pw + dx;
            if (w >= 0 && w < W) m = fmaxf(m, __ldg(xp + (long long)h * W + w));
        }
    }
    Y[idx] = m;
    if (RELU_OUT) Yr[idx] = fmaxf(rs ? fmaf(m, __ldg(rs + (int)(pl % C)), __ldg(rb + (int)(pl % C))) : m, 0.f);
}

// Channels-last input (B,H,W,C), NCHW output: what follows a convolution that runs channels-last (the 7x7 stem is
// fastest that way) when the next layer wants NCHW.  A block takes one output row of 32 * VEC channels: lanes run along
// the channels for the loads (VEC = 2: 256 contiguous bytes per pixel and warp, so that with 64 channels a warp walks
// whole input rows), the row is turned through shared memory, and lanes run along the pixels for the stores.
template <int VEC, bool RELU_OUT>
__global__ void __launch_bounds__(256) maxpool_nhwc_in_kernel(const float *__restrict__ X, float *__restrict__ Y, float *__restrict__ Yr,
                                                                const float *__restrict__ rs, const float *__restrict__ rb, int C, int H,
                                                                int W, int OH, int OW, int ph, int pw, int pitch)
{
    constexpr int CB = 32 * VEC;
    extern __shared__ float S[];                    // [CB channels][pitch]
    const int oh = blockIdx.x % OH, b = blockIdx.x / OH;
    const int c0 = blockIdx.y * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool c_ok = c0 + VEC * lane < C;          // (VEC = 2 is used for even C only: the pair is in or out together)
    const float ninf = -__int_as_float(0x7f800000);
    for (int ow = warp; ow < OW; ow += 8) {
        float m0 = ninf, m1 = ninf;
#pragma unroll
        for (int dy = 0; dy < 3; ++dy) {
            const int h = 2 * oh - ph + dy;
            if (h < 0 || h >= H) continue;
#pragma unroll
            for (int dx = 0; dx < 3; ++dx) {
                const int w = 2 * ow - pw + dx;
                if (w >= 0 && w < W && c_ok) {
                    const float *p = X + (((long long)b * H + h) * W + w) * C + c0 + VEC * lane;
                    if (VEC == 2) { const float2 v = __ldg(reinterpret_cast<const float2 *>(p)); m0 = fmaxf(m0, v.x); m1 = fmaxf(m1, v.y); }
                    else m0 = fmaxf(m0, __ldg(p));
                }
            }
        }
        S[(VEC * lane) * pitch + ow] = m0;
        if (VEC == 2) S[(VEC * lane + 1) * pitch + ow] = m1;
    }
    __syncthreads();
    for (int c = warp; c < CB && c0 + c < C; c += 8) {
        const long long o = (((long long)b * C + c0 + c) * OH + oh) * OW;
        const float sc = (RELU_OUT && rs) ? __ldg(rs + c0 + c) : 1.f, sh = (RELU_OUT && rs) ? __ldg(rb + c0 + c) : 0.f;
        for (int ow = lane; ow < OW; ow += 32) {
            const float v = S[c * pitch + ow];
            Y[o + ow] = v;
            if (RELU_OUT) Yr[o + ow] = fmaxf(fmaf(v, sc, sh), 0.f);
        }
    }
}

int maxpool3x3s2_same_nhwc_in(const float *X, float *Y, float *Yrelu, const float *rs, const float *rb, int B, int C, int H, int W,
                              cudaStream_t st)
{
    if (!X || !Y || B <= 0 || C <= 0 || H <= 0 || W <= 0) return WG2X2_ERR_BAD_ARG;
    if ((rs == nullptr) != (rb == nullptr) || (rs && !Yrelu)) return WG2X2_ERR_BAD_ARG;
    const int OH = (H + 1) / 2, OW = (W + 1) / 2, ph = H & 1, pw = W & 1;
    const int pitch = OW | 1;
    const bool vec2 = (C % 2 == 0) && C >= 64 && (reinterpret_cast<uintptr_t>(X) & 7u) == 0;
    const int cb = vec2 ? 64 : 32;
    const size_t smem = (size_t)cb * pitch * sizeof(float);
    if ((long long)B * OH > 0x7fffffffLL || cdiv(C, cb) > 65535 || smem > 48 * 1024) return WG2X2_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)(B * OH), cdiv(C, cb));
#define WG_POOL_LAUNCH(V, R) maxpool_nhwc_in_kernel<V, R><<<grid, 256, smem, st>>>(X, Y, Yrelu, rs, rb, C, H, W, OH, OW, ph, pw, pitch)
    if (vec2) { if (Yrelu) WG_POOL_LAUNCH(2, true); else WG_POOL_LAUNCH(2, false); }
    else      { if (Yrelu) WG_POOL_LAUNCH(1, true); else WG_POOL_LAUNCH(1, false); }
#undef WG_POOL_LAUNCH
    return launch_status();
}

int maxpool3x3s2_same(const float *X, float *Y, float *Yrelu, const float *rs, const float *rb, int B, int C, int H, int W,
                      cudaStream_t st)
{
    if (!X || !Y || B <= 0 || C <= 0 || H <= 0 || W <= 0) return WG2X2_ERR_BAD_ARG;
    if ((rs == nullptr) != (rb == nullptr) || (rs && !Yrelu)) return WG2X2_ERR_BAD_ARG;
    const int OH = (H + 1) / 2, OW = (W + 1) / 2, ph = H & 1, pw = W & 1;
    const long long planes = (long long)B * C;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if ((W % 8) == 0 && al16(X) && al16(Y) && (!Yrelu || al16(Yrelu))) {
        const long long total = planes * OH * (OW / 4);
        const long long blocks = cdivll(total, 256);
        if (blocks > 0x7fffffffLL) return WG2X2_ERR_UNSUPPORTED;
        if (Yrelu) maxpool_vec_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph);
        else       maxpool_vec_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph);
    } else if ((W % 4) == 0 && al16(X) && al16(Y) && (!Yrelu || al16(Yrelu))) {
        const long long total = planes * OH * (OW / 2);
        const long long blocks = cdivll(total, 256);
        if (blocks > 0x7fffffffLL) return WG2X2_ERR_UNSUPPORTED;
        if (Yrelu) maxpool_vec2_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph);
        else       maxpool_vec2_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph);
    } else {
        const long long blocks = cdivll(planes * OH * OW, 256);
        if (blocks > 0x7fffffffLL) return WG2X2_ERR_UNSUPPORTED;
        if (Yrelu) maxpool_any_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph, pw);
        else       maxpool_any_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(X, Y, Yrelu, rs, rb, C, planes, H, W, OH, OW, ph, pw);
    }
    return launch_status();
}

}  // namespace wg

extern "C" int wg2x2_maxpool3x3s2_same_nhwc_in(const float *X, float *Y, float *Y_relu, const float *relu_scale, const float *relu_shift,
                                               int B, int C, int H, int W, void *stream)
{
    return wg::maxpool3x3s2_same_nhwc_in(X, Y, Y_relu, relu_scale, relu_shift, B, C, H, W, (cudaStream_t)stream);
}

extern "C" int wg2x2_maxpool3x3s2_same(const float *X, float *Y, float *Y_relu, const float *relu_scale, const float *relu_shift,
                                       int B, int C, int H, int W, void *stream)
{
    return wg::maxpool3x3s2_same(X, Y, Y_relu, relu_scale, relu_shift, B, C, H, W, (cudaStream_t)stream);
}
