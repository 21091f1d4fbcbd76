// The dense head of the reference's ResNet-18-var graph in one kernel: the 7x7 / stride 2 convolution of the
// 3-channel image into 64 channels (Conv2D('conv1', image, 64, 7, stride=2), no bias, no activation) followed by
// the 3x3 / stride 2 max-pool ('pool1'), both with TensorFlow's SAME padding
// (ResNet-18-var/imagenet-resnet-transWino-prune.py:112-114), and optionally relu(scale * pooled + shift), the
// BNReLU the first stage's shortcut starts from (:126-127).  The reference leaves this layer dense; it is here
// because a stock convolution of a 3-channel image costs more than all sixteen Winograd layers together, and
// because fusing the pool keeps the (B,64,H/2,W/2) convolution result, the largest tensor of the network, out of
// memory altogether.
//
// Method: implicit GEMM on the warp-level tensor-core path (mma.sync m16n8k8, TF32 operands, FP32 accumulate).
// One block owns a band of pooled rows of one image and walks down it two convolution rows at a time:
//   * the nine image rows those two convolution rows read are staged in shared memory (cp.async, double buffered,
//     zero rows and columns standing for the padding), and A fragments are read straight from that staging with a
//     per-k offset table: no im2col buffer exists anywhere;
//   * warp w owns output columns 16w .. 16w+15 of both rows for all 64 channels (2 x 8 accumulator tiles), so the
//     vertical maximum of a pool window is taken between its own registers; the row shared with the previous step
//     is parked in tensor memory meanwhile (tcgen05.st / tcgen05.ld of the 32 accumulator registers, 64 columns per
//     block: registers are what limits the MMA loop, and tensor memory is otherwise idle here), and the horizontal
//     maximum needs one value per output from the neighbouring column pair, exchanged through shared memory;
//   * the weights are pre-rounded to TF32 and pre-arranged so that a lane fetches its sixteen B values of a k-step
//     with four 16-byte loads.
// K runs over the 21 (ky, channel) pairs times 8: the seven taps of a kernel row and a zero weight, so that every
// k-step reads eight consecutive staged pixels at an offset known at compile time.  Image values are rounded to
// TF32 (nearest) on the fly.
//
// Why the warp-level MMA and not tcgen05 here: with three input channels the A operand is an im2col view that no
// TMA box can produce, so a shared-memory-operand MMA would need the threads to build a swizzled [128 x 168] tile
// per 128 pixels first, which moves as many shared-memory bytes as the register fragments do now.  The kernel is
// bound by that operand traffic (about 3 KB per 16 MMAs and warp) together with the MMA issue rate (8 clocks per
// m16n8k8 and SM sub-partition, 271 TFLOP/s over the chip): it reaches about half of that rate.
#include "wg_common.cuh"

namespace wg {

constexpr int kStemThreads = 224;       // 7 warps x 16 output columns = 112 = the widest row handled
constexpr int kStemPitch = 232;         // staged row: 4 zeros, up to 224 pixels, 4 zeros
constexpr int kStemRows = 9;            // image rows under two consecutive convolution rows
constexpr int kStemKSteps = 21;         // one per (ky, channel): k = 8*(3*ky + c) + kx, kx = 7 carrying a zero weight
constexpr int kStemBuf = 3 * kStemRows * kStemPitch;
constexpr int kStemWt = kStemKSteps * 32 * 16;
constexpr int kStemEPitch = 60;
constexpr int kStemMaxW = 224;

struct StemSmem {
    float wt[kStemWt];
    float in[2][kStemBuf];
    float e[64 * kStemEPitch];
    float2 affine[64];                   // scale and shift of the ReLU output per channel
    uint32_t tmem_base;                  // written by tcgen05.alloc
};

constexpr uint32_t kStemTmemCols = 64;   // warps 0..3 park their row in columns 0..31 of their 32 lanes, warps 4..6 in 32..63

__device__ __forceinline__ void stem_tmem_st32(uint32_t taddr, const float (&r)[8][4])
{
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"r"(taddr + 8 * q), "r"(__float_as_uint(r[2 * q][0])), "r"(__float_as_uint(r[2 * q][1])),
                       "r"(__float_as_uint(r[2 * q][2])), "r"(__float_as_uint(r[2 * q][3])), "r"(__float_as_uint(r[2 * q + 1][0])),
                       "r"(__float_as_uint(r[2 * q + 1][1])), "r"(__float_as_uint(r[2 * q + 1][2])), "r"(__float_as_uint(r[2 * q + 1][3]))
                     : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void stem_tmem_ld32(uint32_t taddr, float (&r)[8][4])
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t u[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7])
                     : "r"(taddr + 8 * q) : "memory");
#pragma unroll
        for (int e = 0; e < 8; ++e) r[2 * q + (e >> 2)][e & 3] = __uint_as_float(u[e]);
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// (64,3,7,7) weights -> [k-step][4][lane][4]: a lane's sixteen values e = 4*quad + comp are B fragment register 0
// (k = 8*ks + t) of the eight 8-channel tiles for e < 8, register 1 (k = 8*ks + t + 4) for e >= 8, channel
// 8*(e%8) + g; lane = 4*g + t.  Each quad is one 16-byte load, contiguous over the lanes (no bank conflicts).
// k = 8*(3*ky + c) + kx.
__global__ void stem_prepare_kernel(const float *__restrict__ W, float *__restrict__ Wp)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= kStemWt) return;
    const int e = ((idx >> 7) & 3) * 4 + (idx & 3), lane = (idx >> 2) & 31, ks = idx >> 9;
    const int g = lane >> 2, t = lane & 3;
    const int k = 8 * ks + t + 4 * (e >> 3), n = 8 * (e & 7) + g;
    float v = 0.f;
    if ((k & 7) < 7) {
        const int ky = (k >> 3) / 3, c = (k >> 3) % 3, kx = k & 7;
        v = W[((n * 3 + c) * 7 + ky) * 7 + kx];
    }
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    Wp[idx] = __uint_as_float(r);
}

__device__ __forceinline__ uint32_t to_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Accumulate convolution rows r1 (acc[0], only if BOTH) and r1+1 (acc[1]) from a staged buffer whose row y holds
// image row 2*r1 - 2 + y.  Tile row g is output column 16w + 2g, tile row g + 8 the column after it: with that
// order the lanes of an A load are 4 floats apart per g and 1 per t, one bank each.
template <bool BOTH>
__device__ __forceinline__ void stem_rows(const float *__restrict__ S, const float4 *__restrict__ wt4, int lane, int warp,
                                          float (&acc)[2][8][4])
{
    const int g = lane >> 2, t = lane & 3;
    const float *p0 = S + 32 * warp + 4 * g + 2 + t;  // column 2*ow - 2 of the image = staged index 2*ow + 2
    const float *p1 = p0 + 2 * kStemPitch;
    const float4 *q = wt4 + lane;
#pragma unroll
    for (int ks = 0; ks < kStemKSteps; ++ks) {
        const int off = ((ks % 3) * kStemRows + ks / 3) * kStemPitch;   // staged row of (channel, ky)
        const float4 q0 = q[ks * 128], q1 = q[ks * 128 + 32], q2 = q[ks * 128 + 64], q3 = q[ks * 128 + 96];
        const uint32_t b0[8] = {__float_as_uint(q0.x), __float_as_uint(q0.y), __float_as_uint(q0.z), __float_as_uint(q0.w),
                                __float_as_uint(q1.x), __float_as_uint(q1.y), __float_as_uint(q1.z), __float_as_uint(q1.w)};
        const uint32_t b1[8] = {__float_as_uint(q2.x), __float_as_uint(q2.y), __float_as_uint(q2.z), __float_as_uint(q2.w),
                                __float_as_uint(q3.x), __float_as_uint(q3.y), __float_as_uint(q3.z), __float_as_uint(q3.w)};
        uint32_t a1[4] = {to_tf32(p1[off]), to_tf32(p1[off + 2]), to_tf32(p1[off + 4]), to_tf32(p1[off + 6])};
        uint32_t a0[4];
        if (BOTH) {
            a0[0] = to_tf32(p0[off]); a0[1] = to_tf32(p0[off + 2]); a0[2] = to_tf32(p0[off + 4]); a0[3] = to_tf32(p0[off + 6]);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mma_tf32(acc[1][nt], a1, b0[nt], b1[nt]);
            if (BOTH) mma_tf32(acc[0][nt], a0, b0[nt], b1[nt]);
        }
    }
}

// Stage the nine image rows 2*r1 - 2 .. 2*r1 + 6 of the three channels; rows outside the image become zeros.
// Warp w takes staged rows w, w+7, w+14, w+21 of the 27, its lanes the 16-byte pieces of a row (two passes).
__device__ __forceinline__ void stem_stage(float *buf, const float *__restrict__ img, int r1, int H, int W, int lane, int warp)
{
    const int W4 = W >> 2;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = warp + 7 * it;
        if (r < 3 * kStemRows) {
            const int c = r / kStemRows, y = r - c * kStemRows;
            const int row = 2 * r1 - 2 + y;
            float *dst = buf + r * kStemPitch + 4 + 4 * lane;
            if (row >= 0 && row < H) {
                const float *src = img + ((long long)c * H + row) * W + 4 * lane;
                const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
                if (lane < W4) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
                if (lane + 32 < W4) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d + 512), "l"(src + 128) : "memory");
            } else {
                if (lane < W4) *reinterpret_cast<float4 *>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                if (lane + 32 < W4) *reinterpret_cast<float4 *>(dst + 128) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <bool RELU_OUT>
__global__ void __launch_bounds__(kStemThreads, 2)
stem_pool_kernel(const float *__restrict__ X, const float *__restrict__ Wp, float *__restrict__ Y, float *__restrict__ Yr,
                 const float *__restrict__ rs, const float *__restrict__ rb, int H, int W, int bands, int band_rows)
{
    extern __shared__ __align__(16) unsigned char stem_smem_raw[];
    StemSmem &sm = *reinterpret_cast<StemSmem *>(stem_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / bands, band = blockIdx.x % bands;
    const int OH = H >> 1, OW = W >> 1, PH = OH >> 1, PW = OW >> 1;
    const int pr0 = band * band_rows, pr1 = min(PH, pr0 + band_rows);
    const float *img = X + (long long)b * 3 * H * W;

    // zero both staging buffers (padding columns stay zero for the whole kernel), fetch the weights
    for (int i = tid; i < 2 * kStemBuf / 4; i += kStemThreads) reinterpret_cast<float4 *>(&sm.in[0][0])[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = tid; i < kStemWt / 4; i += kStemThreads) reinterpret_cast<float4 *>(sm.wt)[i] = __ldg(reinterpret_cast<const float4 *>(Wp) + i);
    if (tid < 64) sm.affine[tid] = rs ? make_float2(__ldg(rs + tid), __ldg(rb + tid)) : make_float2(1.f, 0.f);
    if (warp == 0) {     // two blocks of this kernel share an SM's 512 columns: the allocation never has to wait
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(&sm.tmem_base)), "r"(kStemTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // a warp reaches the 32 tensor-memory lanes of its quarter (warp % 4) only
    const uint32_t tcarry = sm.tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * 32);

    const int nsteps = pr1 - pr0 + 1;                  // step 0 computes convolution row 2*pr0 alone
    stem_stage(sm.in[0], img, 2 * pr0 - 1, H, W, lane, warp);

    const int g = lane >> 2, t = lane & 3;
    const int j = 8 * warp + g;                        // pooled column of this lane
    const bool col_ok = j < PW;
    for (int s = 0; s < nsteps; ++s) {
        const int i = pr0 + s - 1;                     // pooled row this step completes (s >= 1)
        if (s + 1 < nsteps) {
            stem_stage(sm.in[(s + 1) & 1], img, 2 * (pr0 + s) + 1, H, W, lane, warp);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float acc[2][8][4];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][nt][e] = 0.f;
        if (s == 0) {
            stem_rows<false>(sm.in[0], reinterpret_cast<const float4 *>(sm.wt), lane, warp, acc);
            stem_tmem_st32(tcarry, acc[1]);
        } else {
            stem_rows<true>(sm.in[s & 1], reinterpret_cast<const float4 *>(sm.wt), lane, warp, acc);
            const bool low_ok = 2 * i + 2 < OH;        // the window's third row exists
            float carry[8][4];                         // convolution row 2*i, computed by the previous step
            stem_tmem_ld32(tcarry, carry);
            stem_tmem_st32(tcarry, acc[1]);
            float h[8][2];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[e] = fmaxf(carry[nt][e], acc[0][nt][e]);
                    if (low_ok) v[e] = fmaxf(v[e], acc[1][nt][e]);
                }
                h[nt][0] = fmaxf(v[0], v[2]);
                h[nt][1] = fmaxf(v[1], v[3]);
                if (col_ok) {
                    sm.e[(8 * nt + 2 * t) * kStemEPitch + j] = v[0];
                    sm.e[(8 * nt + 2 * t + 1) * kStemEPitch + j] = v[1];
                }
            }
            __syncthreads();
            if (col_ok) {
                const bool right_ok = 2 * j + 2 < OW;
                const long long plane = (long long)PH * PW;
                const long long base = ((long long)b * 64 + 2 * t) * plane + (long long)i * PW + j;
                const float *ep = sm.e + 2 * t * kStemEPitch + j + 1;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        float o = h[nt][c];
                        if (right_ok) o = fmaxf(o, ep[(8 * nt + c) * kStemEPitch]);
                        const long long off = base + (8 * nt + c) * plane;
                        Y[off] = o;
                        if (RELU_OUT) {
                            const float2 af = sm.affine[8 * nt + 2 * t + c];
                            Yr[off] = fmaxf(fmaf(o, af.x, af.y), 0.f);
                        }
                    }
            }
        }
        __syncthreads();   // the buffer just read is staged into at the top of the next step; e[] is rewritten
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(kStemTmemCols) : "memory");
    }
}

int stem_prepare(const float *W, float *Wp, cudaStream_t st)
{
    if (!W || !Wp) return WG2X2_ERR_BAD_ARG;
    stem_prepare_kernel<<<cdiv(kStemWt, 256), 256, 0, st>>>(W, Wp);
    return launch_status();
}

int stem_pool(const float *X, const float *Wp, float *Y, float *Yrelu, const float *rs, const float *rb, int B, int H, int W,
              cudaStream_t st)
{
    if (!X || !Wp || !Y || B <= 0) return WG2X2_ERR_BAD_ARG;
    if ((rs == nullptr) != (rb == nullptr) || (rs && !Yrelu)) return WG2X2_ERR_BAD_ARG;
    if (H < 4 || W < 4 || (H & 3) || (W & 3)) return WG2X2_ERR_UNSUPPORTED;   // even convolution and pool sizes only
    if (W > kStemMaxW) return WG2X2_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (reinterpret_cast<uintptr_t>(Wp) & 15u)) return WG2X2_ERR_BAD_ARG;
    const int PH = H / 4;
    // bands of pooled rows per block: every band recomputes one convolution row (about half a step), and the blocks
    // run in waves of two per SM; take the band height with the least rows-in-flight per SM over the whole launch
    int band_rows = PH;
    double best = 1e30;
    for (int r = 1; r <= PH; ++r) {
        const long long n = (long long)B * cdiv(PH, r);
        const double cost = (double)cdivll(n, 2 * kNumSMs) * (r + 0.55);
        if (cost < best) { best = cost; band_rows = r; }
    }
    const int bands = cdiv(PH, band_rows);
    const long long blocks = (long long)B * bands;
    if (blocks > 0x7fffffffLL) return WG2X2_ERR_UNSUPPORTED;
    const size_t smem = sizeof(StemSmem);
    if (Yrelu) {
        if (cudaFuncSetAttribute(stem_pool_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(stem_pool_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        stem_pool_kernel<true><<<(unsigned)blocks, kStemThreads, smem, st>>>(X, Wp, Y, Yrelu, rs, rb, H, W, bands, band_rows);
    } else {
        if (cudaFuncSetAttribute(stem_pool_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(stem_pool_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        stem_pool_kernel<false><<<(unsigned)blocks, kStemThreads, smem, st>>>(X, Wp, Y, Yrelu, rs, rb, H, W, bands, band_rows);
    }
    return launch_status();
}

}  // namespace wg

extern "C" int wg2x2_stem_prepared_floats(void) { return wg::kStemWt; }

extern "C" int wg2x2_stem_prepare(const float *W, float *Wp, void *stream) { return wg::stem_prepare(W, Wp, (cudaStream_t)stream); }

extern "C" int wg2x2_stem7x7s2_pool(const float *X, const float *Wp, float *Y, float *Y_relu, const float *relu_scale,
                                    const float *relu_shift, int B, int H, int W, void *stream)
{
    return wg::stem_pool(X, Wp, Y, Y_relu, relu_scale, relu_shift, B, H, W, (cudaStream_t)stream);
}
