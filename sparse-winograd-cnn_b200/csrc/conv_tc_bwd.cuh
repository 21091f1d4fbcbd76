// Tensor-core gradient products.  Included by conv_tc.cu (same translation unit: the kernels share the
// PTX wrappers, the status word and the plane-mode instantiation of the tcgen05 kernel).
//
//   dM  = A dY A^T           conv_dm_*_kernel: one HBM-bound pass, 16 planes [t][P][K], rounded to TF32
//   dV_t = dM_t . W_t^T      conv_grad_gemm_tc_kernel<1> (A = dM, B = W as stored: (16,C,K) is already
//                            contraction-contiguous for this product), ReLU mask in the epilogue
//   dW_t = V_t^T . dM_t      conv_grad_gemm_tc_kernel<0> (both operands MN-major), split over P
#pragma once

static inline bool misaligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }   // NULL passes

// ---------------------------------------------------------------------------------------
// dM producer
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float round_tf32(float x)
{
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

// NHWC: one thread = one tile x 4 output channels
__global__ void __launch_bounds__(256) conv_dm_nhwc_kernel(const float *__restrict__ dY, float *__restrict__ dM, long long P, int nH,
                                                             int nW, int H, int W, int K)
{
    const int KV = K >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P * KV) return;
    const int kv = (int)(idx % KV);
    const long long p = idx / KV;
    const int tw = (int)(p % nW), th = (int)((p / nW) % nH), b = (int)(p / ((long long)nW * nH));
    float4 g[2][2];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int h = 2 * th + a, w = 2 * tw + e;
            g[a][e] = (h < H && w < W) ? __ldg(reinterpret_cast<const float4 *>(dY + (((long long)b * H + h) * W + w) * K) + kv)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    float m0[4][4], m1[4][4], m2[4][4], m3[4][4];
    a_g_at(g[0][0].x, g[0][1].x, g[1][0].x, g[1][1].x, m0);
    a_g_at(g[0][0].y, g[0][1].y, g[1][0].y, g[1][1].y, m1);
    a_g_at(g[0][0].z, g[0][1].z, g[1][0].z, g[1][1].z, m2);
    a_g_at(g[0][0].w, g[0][1].w, g[1][0].w, g[1][1].w, m3);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            reinterpret_cast<float4 *>(dM + ((long long)(4 * i + j) * P + p) * K)[kv] =
                make_float4(round_tf32(m0[i][j]), round_tf32(m1[i][j]), round_tf32(m2[i][j]), round_tf32(m3[i][j]));
}

// NCHW: a CTA stages a band of 2R rows of dY for 32 channels (one contiguous run per channel), then walks
// tiles with lane = channel so that the plane stores are contiguous along K.  Any layout/width: R >= 1.
__global__ void __launch_bounds__(256) conv_dm_nchw_kernel(const float *__restrict__ dY, float *__restrict__ dM, long long P, int nH,
                                                             int nW, int H, int W, int K, int R, int nbands, int pitch)
{
    extern __shared__ float S[];
    const int band = blockIdx.x % nbands;
    const int b = blockIdx.x / nbands;
    const int k0 = blockIdx.y * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int th0 = band * R;
    const int rows_tile = min(R, nH - th0);
    const int lo = 2 * th0, hi = min(2 * th0 + 2 * rows_tile, H);
    const int nfill = (hi - lo) * W;
    for (int kk = warp; kk < 32; kk += 8) {
        if (k0 + kk >= K) break;
        const float *src = dY + (((long long)b * K + k0 + kk) * H + lo) * W;
        float *dst = S + kk * pitch;
        for (int i = lane; i < nfill; i += 32) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    if (k0 + lane >= K) return;
    const float *Sk = S + lane * pitch;
    for (int q = warp; q < rows_tile * nW; q += 8) {
        const int tr = q / nW, tw = q - tr * nW;
        float g[2][2];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = lo + 2 * tr + a, w = 2 * tw + e;
                g[a][e] = (h < H && w < W) ? Sk[(2 * tr + a) * W + w] : 0.f;
            }
        float m[4][4];
        a_g_at(g[0][0], g[0][1], g[1][0], g[1][1], m);
        const long long p = ((long long)b * nH + th0 + tr) * nW + tw;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) dM[((long long)(4 * i + j) * P + p) * K + k0 + lane] = round_tf32(m[i][j]);
    }
}

// The same with four channels per lane: 16-byte plane stores, 512 bytes per warp and store with LC = 32 lanes along
// the channels (128 per CTA; LC = 16 would be 64 per CTA, the two halves of a warp on two tiles at once -- not used:
// it measured slower than one channel per lane).  Where the band is the whole image, the CTA's channels are one
// contiguous run of dY and are staged as such.
template <int LC>
__global__ void __launch_bounds__(256, 3) conv_dm_nchw_vec_kernel(const float *__restrict__ dY, float *__restrict__ dM, long long P, int nH,
                                                                    int nW, int H, int W, int K, int R, int nbands, int pitch)
{
    constexpr int CB = 4 * LC, QW = 32 / LC;
    extern __shared__ float S[];
    const int band = blockIdx.x % nbands;
    const int b = blockIdx.x / nbands;
    const int k0 = blockIdx.y * CB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lc = lane % LC, lq = lane / LC;
    const int th0 = band * R;
    const int rows_tile = min(R, nH - th0);
    const int lo = 2 * th0, hi = min(2 * th0 + 2 * rows_tile, H);
    const int nfill = (hi - lo) * W;
    const int nch = min(CB, K - k0);
    if (nfill == H * W) {
        const float *src = dY + ((long long)b * K + k0) * nfill;
        for (int k = threadIdx.x; k < nch * nfill; k += 256) {
            const int kk = k / nfill;
            S[kk * pitch + (k - kk * nfill)] = __ldg(src + k);
        }
    } else {
        for (int kk = warp; kk < nch; kk += 8) {
            const float *src = dY + (((long long)b * K + k0 + kk) * H + lo) * W;
            float *dst = S + kk * pitch;
            for (int i = lane; i < nfill; i += 32) dst[i] = __ldg(src + i);
        }
    }
    __syncthreads();
    if (k0 + 4 * lc >= K) return;
    const float *Sk = S + 4 * lc * pitch;
#pragma unroll 1
    for (int q = warp * QW + lq; q < rows_tile * nW; q += 8 * QW) {
        const int tr = q / nW, tw = q - tr * nW;
        float g[4][2][2];
#pragma unroll
        for (int v = 0; v < 4; ++v)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int h = lo + 2 * tr + a, w = 2 * tw + e;
                    g[v][a][e] = (h < H && w < W) ? Sk[v * pitch + (2 * tr + a) * W + w] : 0.f;
                }
        float m0[4][4], m1[4][4], m2[4][4], m3[4][4];
        a_g_at(g[0][0][0], g[0][0][1], g[0][1][0], g[0][1][1], m0);
        a_g_at(g[1][0][0], g[1][0][1], g[1][1][0], g[1][1][1], m1);
        a_g_at(g[2][0][0], g[2][0][1], g[2][1][0], g[2][1][1], m2);
        a_g_at(g[3][0][0], g[3][0][1], g[3][1][0], g[3][1][1], m3);
        const long long p = ((long long)b * nH + th0 + tr) * nW + tw;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<float4 *>(dM + ((long long)(4 * i + j) * P + p) * K + k0 + 4 * lc) =
                    make_float4(round_tf32(m0[i][j]), round_tf32(m1[i][j]), round_tf32(m2[i][j]), round_tf32(m3[i][j]));
    }
}

// W (16, C, K) -> W rounded to TF32, plus the zero-block map of the forward's prepared weights: bit cc of
// map[t][kb] is set when the block (input channels cc*32.., output channels kb*64..) holds a non-zero.
// One CTA per block: 32 rows of 64 consecutive floats.
__global__ void __launch_bounds__(256) round_and_map_kernel(const float *__restrict__ Wt, float *__restrict__ Wr,
                                                              unsigned long long *__restrict__ map, int C, int K, int nKB, int nCC)
{
    const int kb = blockIdx.x, cc = blockIdx.y, t = blockIdx.z;
    int nz = 0;
    if ((K & 3) == 0 && ((reinterpret_cast<uintptr_t>(Wt) | reinterpret_cast<uintptr_t>(Wr)) & 15u) == 0) {
        // 16 bytes per access: 32 rows of 16 float4, two per thread
#pragma unroll
        for (int e = threadIdx.x; e < 32 * 16; e += 256) {
            const int c = cc * 32 + (e >> 4), k = kb * 64 + 4 * (e & 15);
            if (c < C && k < K) {
                const long long o = ((long long)t * C + c) * K + k;
                float4 w = __ldg(reinterpret_cast<const float4 *>(Wt + o));
                w.x = round_tf32(w.x); w.y = round_tf32(w.y); w.z = round_tf32(w.z); w.w = round_tf32(w.w);
                *reinterpret_cast<float4 *>(Wr + o) = w;
                nz |= (w.x != 0.f) | (w.y != 0.f) | (w.z != 0.f) | (w.w != 0.f);
            }
        }
    } else {
        for (int e = threadIdx.x; e < 32 * 64; e += 256) {
            const int c = cc * 32 + (e >> 6), k = kb * 64 + (e & 63);
            if (c < C && k < K) {
                const long long o = ((long long)t * C + c) * K + k;
                const float w = round_tf32(__ldg(Wt + o));
                Wr[o] = w;
                nz |= (w != 0.f);
            }
        }
    }
    nz = __syncthreads_or(nz);
    if (threadIdx.x == 0 && nz && nCC <= 64) atomicOr(map + (long long)t * nKB + kb, 1ull << cc);
}

static int launch_dm(const float *dY, float *dM, int B, int H, int W, int K, int layout, cudaStream_t st)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const long long P = (long long)B * nH * nW;
    if (layout == WG2X2_NHWC) {
        conv_dm_nhwc_kernel<<<(unsigned)cdivll(P * (K / 4), 256), 256, 0, st>>>(dY, dM, P, nH, nW, H, W, K);
    } else if (K % 4 == 0 && K >= 128 && 2 * nH * W <= 96 && (reinterpret_cast<uintptr_t>(dM) & 15u) == 0 &&
               (long long)B * cdiv(K, 128) >= 4LL * kNumSMs) {
        // Four channels per lane, 128 per CTA, where the whole image is one small band and the CTAs fill the GPU
        // (256 x 512 x 7 x 7: the backward step 193 against 197 us).  With several bands per image, or 64 channels
        // per CTA, the one-channel-per-lane kernel below measured faster (144 against 161 us at 14 x 14).
        const int R = nH, nbands = 1;
        const int pitch = (2 * R * W) | 1;
        const int smem = 128 * pitch * (int)sizeof(float);
        if ((long long)B > 0x7fffffffLL || cdiv(K, 128) > 65535) return WG2X2_ERR_UNSUPPORTED;
        const dim3 grid((unsigned)B, cdiv(K, 128));
        if (cudaFuncSetAttribute(conv_dm_nchw_vec_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        conv_dm_nchw_vec_kernel<32><<<grid, 256, smem, st>>>(dY, dM, P, nH, nW, H, W, K, R, nbands, pitch);
    } else {
        int R = 384 / (2 * W);
        if (R < 1) R = 1;
        if (R > nH) R = nH;
        const int nbands = cdiv(nH, R);
        const int pitch = (2 * R * W) | 1;
        const int smem = 32 * pitch * (int)sizeof(float);
        if ((long long)B * nbands > 0x7fffffffLL || smem > 200 * 1024) return WG2X2_ERR_UNSUPPORTED;
        if (cudaFuncSetAttribute(conv_dm_nchw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        conv_dm_nchw_kernel<<<dim3((unsigned)(B * nbands), cdiv(K, 32)), 256, smem, st>>>(dY, dM, P, nH, nW, H, W, K, R, nbands, pitch);
    }
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// Workspace of the tensor-core backward pass: [dM | W rounded to TF32 | dW partials]
// ---------------------------------------------------------------------------------------
struct BwdWs {
    size_t dm, wr, map, partial, total;
};
static BwdWs bwd_ws_layout(long long P, int C, int K, int dw_splits)
{
    BwdWs w;
    w.dm = 0;
    size_t off = align_up((size_t)16 * P * K * sizeof(float), 256);
    w.wr = off;      off += align_up((size_t)16 * C * K * sizeof(float), 256);
    w.map = off;     off += align_up((size_t)16 * cdiv(K, 64) * sizeof(unsigned long long), 256);
    w.partial = off; off += dw_splits > 1 ? align_up((size_t)dw_splits * 16 * C * K * sizeof(float), 256) : 0;
    w.total = off;
    return w;
}

bool tc_bwd_shape_supported(int C, int K) { return C % 4 == 0 && K % 4 == 0 && C >= 4 && K >= 4; }

// ---------------------------------------------------------------------------------------
// The two gradient products as plain batched GEMMs on the tensor cores (16 independent positions):
//
//   KIND 0   dW_t[c][k] = sum_p V_t[p][c] dM_t[p][k]    rows = C, columns = K, contraction over P (split)
//   KIND 1   dV_t[p][c] = sum_k dM_t[p][k] W_t[c][k]    rows = P, columns = C, contraction over K
//
// Unit = (position t, block of 128 rows, block of N = 64/128/256 columns[, split of the contraction]);
// one fp32 accumulator of N TMEM columns, double-buffered, so the epilogue of a unit overlaps the MMAs of
// the next.  A wide N is what makes these run well: the A tile is read from shared memory and from L2 once
// per 128 x N x 32 products.
//
// KIND 0 operands are stored with the contraction index p as the slow axis, i.e. "MN-major" for UMMA: a
// [32 p x 32 channel] box lands in shared memory as 32 rows of 128 bytes (128B swizzle, 32B atoms), which
// is one MN block of 32 channels x eight K groups of 4 tiles.  A (V_t^T, 128 input channels) is four such
// boxes 4 KB apart (the descriptor's leading-dimension offset), B (dM_t) is N/32 of them.  One MMA (K = 8)
// reads 8 rows: start address + 1024 B per step.
// KIND 1 operands are contraction-contiguous ("K-major"): A = a [128 p x 32 k] box of dM, B = an [N x 32 k]
// box of W exactly as the reference stores it, both with the plain 128B swizzle; + 32 B per MMA step.
//
// The epilogue turns each 32 x 32 block through shared memory so that stores are whole 128-byte lines, and
// applies the pruning mask (KIND 0, one split) or the ReLU mask V > 0 (KIND 1) on the way out.
// ---------------------------------------------------------------------------------------
constexpr int kGgStages = 4;
constexpr int kGgBoxBytes = 32 * 32 * 4;                 // [32 rows][32 fp32]
constexpr int kGgABytes = 4 * kGgBoxBytes;               // 128 rows x 32 contraction steps
constexpr int kGgBBytesMax = 8 * kGgBoxBytes;            // up to 256 columns
constexpr int kGgStageBytes = kGgABytes + kGgBBytesMax;  // 48 KB
constexpr int kGgSmemBytes = kGgStages * kGgStageBytes + 1024 + kCtrlBytes + kEpiWarps * kEpiStageBytes;

struct GgParams {
    float *out;              // [split][16][rows][cols] (split dimension only when !direct)
    const float *mask;       // KIND 0: multiplies the result (direct only); KIND 1: result zeroed where mask <= 0
    long long rows;          // C (KIND 0) or P (KIND 1)
    long long contr;         // P (KIND 0) or K (KIND 1)
    int cols, N;
    int nRB, nCB;
    int splits, chunks_per_split;
    int units;
    int direct;
    // Zero-block skipping (KIND 1 only).  block_map[t][kb] has bit cc set when the 64 x 32 weight block (output
    // channels kb*64.., input channels cc*32..) of position t holds a non-zero (pack_weights_kernel / block_map_kernel).
    //   map_mode 1: columns = output channels, contraction over input channels (forward products)
    //   map_mode 2: columns = input channels, contraction over output channels (dV)
    //   map_mode 0: every chunk runs
    const unsigned long long *block_map;
    int map_mode, map_nkb;
    int tma_out;             // results that need no mask leave by TMA store (mapOut) straight from the staging block
    int mn4;                 // KIND 0: the operand maps are 4-D (channel blocks of 32 as a dimension of their own): one TMA load per operand and chunk
};

// Bit n of the result is set when contraction chunk n (32 elements) of this unit has to run: the first chunk always
// (it zero-initialises the accumulator), a later one unless every weight block it would multiply is all zero.
// Contractions of more than 64 chunks run in full.
__device__ __forceinline__ unsigned long long gg_live_chunks(const GgParams &prm, int t, int cb)
{
    if (prm.map_mode == 0 || prm.contr > 64 * 32) return ~0ull;
    const unsigned long long *row = prm.block_map + (long long)t * prm.map_nkb;
    unsigned long long live = 1ull;
    if (prm.map_mode == 1) {
        const int kb0 = cb * (prm.N >> 6), kb1 = min(prm.map_nkb, kb0 + max(prm.N >> 6, 1));
        for (int kb = kb0; kb < kb1; ++kb) live |= __ldg(row + kb);
    } else {
        const int c0 = cb * (prm.N >> 5), nc = prm.N >> 5;                 // 32-channel chunks covered by this unit's columns
        if (c0 + nc > 64) return ~0ull;
        const unsigned long long sel = (nc >= 64 ? ~0ull : ((1ull << nc) - 1ull)) << c0;
        const int nkb = (int)((prm.contr + 63) >> 6);
        for (int kb = 0; kb < nkb && kb < prm.map_nkb; ++kb)
            if (__ldg(row + kb) & sel) live |= 3ull << (2 * kb);          // both 32-wide halves of the 64-wide block
    }
    return live;
}

// MN-major TF32 operand.  The only shared-memory layout UMMA accepts for it is the 128-byte swizzle with a
// 32-byte base (layout type 1; TMA writes it with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): rows of 128 bytes,
// the 32-byte chunk index XORed with (row & 3), pattern repeating every 4 rows.  MN blocks of 32 elements
// are 4 KB apart (leading-dimension offset), K groups of 4 rows 512 B apart (stride offset).
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(kGgBoxBytes >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

__device__ __forceinline__ void tma_load_4d_gg(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// shared memory -> global, clipped to the tensor; completion is tracked by the thread's bulk async-groups
__device__ __forceinline__ void tma_store_3d(uint32_t src, const CUtensorMap *map, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%1, {%2, %3, %4}], [%0];"
        ::"r"(src), "l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int KIND>
__global__ void __launch_bounds__(kTcThreads, 1)
conv_grad_gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                         const __grid_constant__ CUtensorMap mapOut, const GgParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - raw);
    const uint32_t bars = base + kGgStages * kGgStageBytes;
    uint64_t *bars_gen = reinterpret_cast<uint64_t *>(gen_base + kGgStages * kGgStageBytes);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kGgStages + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * kGgStages + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * kGgStages + 2 + b); };
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bars_gen + 2 * kGgStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_gen + 2 * kGgStages + 5);
    float *epi_stage_all = reinterpret_cast<float *>(gen_base + kGgStages * kGgStageBytes + kCtrlBytes);

    // (broadcast from lane 0: the compiler then treats the warp index, and all that is derived from it, as warp-uniform)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGgStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), kEpiWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_ptr_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_ptr_slot, 0);

    const int N = prm.N;
    // unit -> (split, t, row block, column block); column block fastest so that neighbouring CTAs share the A tile in L2
    auto decode = [&](int u, int &split, int &t, int &rb, int &cb) {
        cb = u % prm.nCB; u /= prm.nCB;
        rb = u % prm.nRB; u /= prm.nRB;
        t = u % 16;
        split = u / 16;
    };

    if (warp == 0) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            const uint32_t stage_tx = (uint32_t)(kGgABytes + N * 128);
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int split, t, rb, cb;
                decode(u, split, t, rb, cb);
                const long long kbeg = (long long)split * prm.chunks_per_split * 32;
                const long long kend = min(prm.contr, kbeg + (long long)prm.chunks_per_split * 32);
                const unsigned long long live = KIND == 1 ? gg_live_chunks(prm, t, cb) : ~0ull;
                for (long long kc = kbeg; kc < kend; kc += 32) {
                    if (KIND == 1 && kc < 64 * 32 && !((live >> (kc >> 5)) & 1ull)) continue;   // all-zero weight blocks: nothing to add
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 0x500u | s)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), stage_tx);
                    const uint32_t a_dst = base + s * kGgStageBytes;
                    const uint32_t b_dst = a_dst + kGgABytes;
                    if (KIND == 0 && prm.mn4) {      // all 32-channel blocks of an operand in one box each
                        tma_load_4d_gg(a_dst, &mapA, full_bar(s), 0, (int)kc, rb * 4, t);
                        tma_load_4d_gg(b_dst, &mapB, full_bar(s), 0, (int)kc, cb * (N / 32), t);
                    } else if (KIND == 0) {
#pragma unroll
                        for (int mb = 0; mb < 4; ++mb)
                            tma_load_3d(a_dst + mb * kGgBoxBytes, &mapA, full_bar(s), rb * 128 + mb * 32, (int)kc, t);
                        for (int nb = 0; nb < N / 32; ++nb)
                            tma_load_3d(b_dst + nb * kGgBoxBytes, &mapB, full_bar(s), cb * N + nb * 32, (int)kc, t);
                    } else {
                        tma_load_3d(a_dst, &mapA, full_bar(s), (int)kc, rb * 128, t);
                        tma_load_3d(b_dst, &mapB, full_bar(s), (int)kc, cb * N, t);
                    }
                    if (++s == kGgStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // The whole warp walks the loop with warp-uniform values (descriptors and addresses in uniform registers); one
        // elected lane issues the MMAs and the commits.  Issued by a lone lane from per-thread registers, an MMA costs
        // several times as many issue slots, for which the eight epilogue warps compete.
        {
            const bool leader = elect_one();
            const uint32_t idesc = make_idesc_tf32(128, N) | (KIND == 0 ? ((1u << 15) | (1u << 16)) : 0u);
            int s = 0; uint32_t ph = 0;
            uint32_t acc_use[2] = {0, 0};
            int buf = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int split, t, rb, cb;
                decode(u, split, t, rb, cb);
                const long long kbeg = (long long)split * prm.chunks_per_split * 32;
                const long long kend = min(prm.contr, kbeg + (long long)prm.chunks_per_split * 32);
                if (!mbar_wait_warp(acce_bar(buf), (acc_use[buf] & 1u) ^ 1u, abort_flag, 0x600u | buf)) { ok = false; break; }
                acc_use[buf]++;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 256);
                uint32_t first = 1;
                const unsigned long long live = KIND == 1 ? gg_live_chunks(prm, t, cb) : ~0ull;
                for (long long kc = kbeg; kc < kend; kc += 32) {
                    if (KIND == 1 && kc < 64 * 32 && !((live >> (kc >> 5)) & 1ull)) continue;
                    if (!mbar_wait_warp(full_bar(s), ph, abort_flag, 0x700u | s)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * kGgStageBytes;
                    const uint64_t adesc = KIND == 0 ? make_desc_mn_sw128(a_addr) : make_desc_k_sw128(a_addr);
                    const uint64_t bdesc = KIND == 0 ? make_desc_mn_sw128(a_addr + kGgABytes) : make_desc_k_sw128(a_addr + kGgABytes);
                    const uint32_t step = KIND == 0 ? 64u : 2u;   // 1024 B / 32 B per 8 contraction steps
                    if (leader) {
#pragma unroll
                        for (int kg = 0; kg < 4; ++kg)
                            umma_tf32(d_tmem, adesc + step * kg, bdesc + step * kg, idesc, (first && kg == 0) ? 0u : 1u);
                        umma_commit(empty_bar(s));
                    }
                    __syncwarp();
                    first = 0;
                    if (++s == kGgStages) { s = 0; ph ^= 1u; }
                }
                if (ok && leader) umma_commit(accf_bar(buf));
                __syncwarp();
                buf ^= 1;
            }
        }
    } else {
        const int ew = warp - 2;
        const int q = warp & 3;
        const int half = ew >> 2;
        float *stg = epi_stage_all + ew * (kEpiStageBytes / 4);
        uint32_t acc_use[2] = {0, 0};
        int buf = 0;
        bool ok = true;
        const long long plane_elems = 16 * prm.rows * prm.cols;
        for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
            int split, t, rb, cb;
            decode(u, split, t, rb, cb);
            const bool use_mask = prm.mask && (KIND == 1 || prm.direct);
            const long long row = (long long)rb * 128 + q * 32 + lane;
            const long long row_off = (prm.direct ? 0 : (long long)split * plane_elems) + ((long long)t * prm.rows + row) * prm.cols;
            const int ncol_half = N / 2;
            // offsets of the 8 lines this lane will store in a 32-column block, and their mask values.  They are fetched one
            // block ahead (the first block of a unit before the accumulator is even waited for), so that the memory latency
            // of the mask hides behind the previous block's TMEM load, turn and stores instead of stalling every block.
            long long off[8], off_nx[8];
            float4 mk[8], mk_nx[8];
            auto fetch = [&](int cc_f, long long (&o)[8], float4 (&m)[8]) {
                const int col_f = cb * N + half * ncol_half + cc_f;
                const long long my_f = (row < prm.rows && col_f < prm.cols) ? row_off + col_f : -1;
                const bool vec_f = (col_f + 32 <= prm.cols) && ((prm.cols & 3) == 0);
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    o[rr] = __shfl_sync(0xffffffffu, my_f, 4 * rr + (lane >> 3));
                    m[rr] = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (vec_f && use_mask && o[rr] >= 0) m[rr] = __ldg(reinterpret_cast<const float4 *>(prm.mask + o[rr] + 4 * (lane & 7)));
                }
            };
            fetch(0, off, mk);
            for (int cc = 0; cc < ncol_half; cc += 32) {
                const int col0 = half * ncol_half + cc;
                const int col = cb * N + col0;
                const long long my_off = (row < prm.rows && col < prm.cols) ? row_off + col : -1;
                const bool vec = (col + 32 <= prm.cols) && ((prm.cols & 3) == 0);
                const bool more = cc + 32 < ncol_half;
                if (more) fetch(cc + 32, off_nx, mk_nx);
                if (cc == 0) {   // first chunk of the unit: only now wait for the accumulator
                    if (!mbar_wait_warp(accf_bar(buf), acc_use[buf] & 1u, abort_flag, 0x800u | (ew << 4) | buf)) { ok = false; break; }
                    acc_use[buf]++;
                    tc_fence_after();
                }
                float r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + col0);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld8(taddr + (uint32_t)(ch * 8), &r[ch * 8]);
                tmem_ld_wait();
                if (vec && prm.tma_out && !use_mask) {
                    // The staging block (32 rows of 128 bytes, 16-byte chunk index XORed with row & 7) is exactly TMA's
                    // 128-byte swizzle: one lane hands it to a TMA store, which also clips the rows beyond the tensor; the
                    // block is not read back through the load/store unit, whose shared-memory traffic competes with the
                    // tensor core's operand reads.  The store that last used the block must have read it first.
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8)
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((c8 ^ (lane & 7)) << 2)) =
                            make_float4(r[4 * c8], r[4 * c8 + 1], r[4 * c8 + 2], r[4 * c8 + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(smem_u32(stg), &mapOut, col, rb * 128 + q * 32, (prm.direct ? 0 : split * 16) + t);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (vec) {
                    if (prm.tma_out) {      // a TMA store of an earlier block may still be reading the staging block
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    __syncwarp();
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8)
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((c8 ^ (lane & 7)) << 2)) =
                            make_float4(r[4 * c8], r[4 * c8 + 1], r[4 * c8 + 2], r[4 * c8 + 3]);
                    __syncwarp();
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        const int srow = 4 * rr + (lane >> 3), ch = lane & 7;
                        float4 v = *reinterpret_cast<const float4 *>(stg + srow * 32 + ((ch ^ (srow & 7)) << 2));
                        if (off[rr] >= 0) {
                            if (KIND == 0) { v.x *= mk[rr].x; v.y *= mk[rr].y; v.z *= mk[rr].z; v.w *= mk[rr].w; }
                            else { v.x = mk[rr].x > 0.f ? v.x : 0.f; v.y = mk[rr].y > 0.f ? v.y : 0.f;
                                   v.z = mk[rr].z > 0.f ? v.z : 0.f; v.w = mk[rr].w > 0.f ? v.w : 0.f; }
                            *reinterpret_cast<float4 *>(prm.out + off[rr] + 4 * ch) = v;
                        }
                    }
                } else if (my_off >= 0) {
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        if (col + x >= prm.cols) continue;
                        float v = r[x];
                        if (use_mask) {
                            const float m1 = __ldg(prm.mask + my_off + x);
                            v = KIND == 0 ? v * m1 : (m1 > 0.f ? v : 0.f);
                        }
                        prm.out[my_off + x] = v;
                    }
                }
                if (more) {
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) { off[rr] = off_nx[rr]; mk[rr] = mk_nx[rr]; }
                }
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(buf));
            buf ^= 1;
        }
        // the last stores must have reached memory before the CTA ends
        if (prm.tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// 3-D map over a (16, rows, ch) fp32 tensor, ch contiguous.  mn_major: box = 32 channels x 32 rows with the
// 32-B-atom 128-B swizzle; otherwise box = 32 channels x box_rows with the plain 128-B swizzle.
static bool make_map_gg(CUtensorMap *map, const float *ptr, long long ch, long long rows, bool mn_major, int box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)ch, (cuuint64_t)rows, 16};
    cuuint64_t strides[2] = {(cuuint64_t)ch * 4, (cuuint64_t)rows * ch * 4};
    cuuint32_t box[3] = {32, (cuuint32_t)(mn_major ? 32 : box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// MN-major operand with the 32-channel blocks as a dimension of their own: (32, rows, ch / 32, 16), box = 32 x 32 rows x
// nblk blocks, which lands in shared memory as nblk consecutive 4 KB blocks -- the layout the MN-major descriptor reads --
// from ONE load instead of nblk.  Needs ch % 32 == 0.
static bool make_map_gg4(CUtensorMap *map, const float *ptr, long long ch, long long rows, int nblk)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || (ch & 31) || nblk < 1 || nblk > 8) return false;
    cuuint64_t dims[4] = {32, (cuuint64_t)rows, (cuuint64_t)(ch / 32), 16};
    cuuint64_t strides[3] = {(cuuint64_t)ch * 4, 128, (cuuint64_t)rows * ch * 4};
    cuuint32_t box[4] = {32, 32, (cuuint32_t)nblk, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int gg_cols(int n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

// Splits of the P range for dW: enough units for every SM, at least 8 chunks of 32 tiles per split
int conv_dw_tc_splits(long long P, int C, int K)
{
    const long long base_units = (long long)16 * cdiv(C, 128) * cdiv(K, gg_cols(K));
    const long long chunks = cdivll(P, 32);
    // one split when the unsplit units already cover most SMs: a second round plus the reduction pass
    // would cost more than the idle SMs do
    long long s = base_units * 3 >= kNumSMs * 2 ? 1 : cdivll(kNumSMs, base_units);
    const long long max_s = chunks / 8 > 0 ? chunks / 8 : 1;
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    const long long cps = cdivll(chunks, s);
    return (int)cdivll(chunks, cps);
}

// 3-D map over the result (planes, rows, cols) fp32, cols contiguous, for the epilogue's TMA stores: box = 32 columns x 32
// rows with the 128-byte swizzle.  Usable when the base is 16-byte aligned and the rows are multiples of 16 bytes.
static bool make_map_out(CUtensorMap *map, float *ptr, long long cols, long long rows, long long planes)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(ptr) & 15u) || (cols & 3)) return false;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)rows * cols * 4};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#include "conv_tc_gemm2.cuh"

// How many pairs of SMs can hold a pair of CTAs of the cta_group::2 kernel at once (0: this device cannot, or
// WG2X2_GEMM_PAIR=0 in the environment); asked once per device and kernel.
template <int KIND>
static int gg_pair_clusters()
{
    static std::atomic<int> cached[64];
    static std::atomic<int> init{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (!init.load()) {
        for (auto &c : cached) c.store(-1);
        init.store(1);
    }
    int n = cached[dev].load();
    if (n >= 0) return n;
    const char *env = getenv("WG2X2_GEMM_PAIR");
    n = 0;
    if (!(env && env[0] == '0') &&
        cudaFuncSetAttribute(conv_grad_gemm_tc2_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGg2SmemBytes) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * kNumSMs);
        cfg.blockDim = dim3(kTcThreads);
        cfg.dynamicSmemBytes = kGg2SmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int got = 0;
        if (cudaOccupancyMaxActiveClusters(&got, conv_grad_gemm_tc2_kernel<KIND>, &cfg) == cudaSuccess && got > 0) n = got;
        else (void)cudaGetLastError();
    }
    cached[dev].store(n);
    return n;
}

// mapB_half: the B operand with boxes of N/2 rows (KIND 1) or N/64 channel blocks (KIND 0, 4-D maps) for the kernel on pairs
// of SMs; NULL: KIND 1 stays on one CTA, KIND 0 loads its 32 x 32 boxes one by one in either kernel.
template <int KIND>
static int gg_launch(const CUtensorMap &mapA, const CUtensorMap &mapB, GgParams &prm, cudaStream_t st, const CUtensorMap *mapB_half = nullptr)
{
    // results without a mask leave by TMA store where the output can be described to TMA (else: the load/store path)
    CUtensorMap mapOut = mapA;
    const bool needs_mask = prm.mask && (KIND == 1 || prm.direct);
    prm.tma_out = (!needs_mask && prm.cols >= 32 &&
                   make_map_out(&mapOut, prm.out, prm.cols, prm.rows, 16LL * (prm.direct ? 1 : prm.splits))) ? 1 : 0;
    // Two SMs per 256 x N tile where that measured faster: long contractions (dW always contracts over all tiles; the
    // products with 512 or more channels), whose pipeline outlasts the pair's extra hand-shakes, and no mask to fetch in
    // the epilogue.  Short contractions (256 channels) and dV with its ReLU mask are HBM-bound and stay on one CTA.
    const bool pair_pays = KIND == 0 ? prm.contr >= 1024 : (mapB_half && prm.contr >= 512 && !needs_mask);
    const int nclusters = (prm.nRB >= 2 && prm.N >= 128 && pair_pays) ? gg_pair_clusters<KIND>() : 0;
    if (nclusters > 0) {
        GgParams p2 = prm;
        p2.nRB = cdiv(prm.nRB, 2);
        p2.units = prm.units / prm.nRB * p2.nRB;
        const int pairs = p2.units < nclusters ? p2.units : nclusters;
        conv_grad_gemm_tc2_kernel<KIND><<<2 * pairs, kTcThreads, kGg2SmemBytes, st>>>(mapA, mapB_half ? *mapB_half : mapB, mapOut, p2);
        return launch_status();
    }
    if (cudaFuncSetAttribute(conv_grad_gemm_tc_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGgSmemBytes) != cudaSuccess)
        return WG2X2_ERR_LAUNCH;
    const int grid = prm.units < kNumSMs ? prm.units : kNumSMs;
    conv_grad_gemm_tc_kernel<KIND><<<grid, kTcThreads, kGgSmemBytes, st>>>(mapA, mapB, mapOut, prm);
    return launch_status();
}

int conv_dw_tc(const float *V, const float *dM, const float *mask, float *dW, float *partial, long long P, int C, int K,
               cudaStream_t st)
{
    GgParams prm;
    prm.rows = C; prm.cols = K; prm.contr = P;
    prm.N = gg_cols(K);
    prm.nRB = cdiv(C, 128);
    prm.nCB = cdiv(K, prm.N);
    prm.splits = conv_dw_tc_splits(P, C, K);
    prm.chunks_per_split = (int)cdivll(cdivll(P, 32), prm.splits);
    prm.units = 16 * prm.nRB * prm.nCB * prm.splits;
    prm.direct = prm.splits == 1;
    prm.out = prm.direct ? dW : partial;
    prm.mask = mask;
    prm.block_map = nullptr; prm.map_mode = 0; prm.map_nkb = 0;
    CUtensorMap mapV, mapM, mapMh;
    prm.mn4 = (C % 32 == 0 && K % 32 == 0) ? 1 : 0;
    if (prm.mn4) {
        if (!make_map_gg4(&mapV, V, C, P, 4) || !make_map_gg4(&mapM, dM, K, P, prm.N / 32) ||
            (prm.N >= 64 && !make_map_gg4(&mapMh, dM, K, P, prm.N / 64)))
            return WG2X2_ERR_LAUNCH;
    } else if (!make_map_gg(&mapV, V, C, P, true, 32) || !make_map_gg(&mapM, dM, K, P, true, 32)) {
        return WG2X2_ERR_LAUNCH;
    }
    const int s = gg_launch<0>(mapV, mapM, prm, st, (prm.mn4 && prm.N >= 64) ? &mapMh : nullptr);
    if (s != WG2X2_OK) return s;
    if (!prm.direct) dw_reduce_launch(partial, mask, dW, (long long)16 * C * K, prm.splits, st);
    return launch_status();
}

int conv_dv_tc(const float *V, const float *Wt, const float *dM, float *Wr, unsigned long long *map, float *dV, long long P, int C,
               int K, int relu, cudaStream_t st)
{
    if (P > 0x7fffffffLL - 128) return WG2X2_ERR_UNSUPPORTED;
    const int nKB = cdiv(K, 64), nCC = cdiv(C, 32);
    if (nCC > 65535) return WG2X2_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(map, nCC <= 64 ? 0 : 0xFF, (size_t)16 * nKB * sizeof(unsigned long long), st) != cudaSuccess) return WG2X2_ERR_LAUNCH;
    round_and_map_kernel<<<dim3(nKB, nCC, 16), 256, 0, st>>>(Wt, Wr, map, C, K, nKB, nCC);
    if (launch_status() != WG2X2_OK) return WG2X2_ERR_LAUNCH;
    GgParams prm;
    prm.rows = P; prm.cols = C; prm.contr = K;
    prm.N = gg_cols(C);
    prm.nRB = (int)cdivll(P, 128);
    prm.nCB = cdiv(C, prm.N);
    prm.splits = 1;
    prm.chunks_per_split = cdiv(K, 32);
    prm.units = 16 * prm.nRB * prm.nCB;
    prm.direct = 1;
    prm.out = dV;
    prm.mask = relu ? V : nullptr;
    prm.block_map = map; prm.map_mode = 2; prm.map_nkb = nKB; prm.mn4 = 0;
    CUtensorMap mapA, mapB, mapBh;
    if (!make_map_gg(&mapA, dM, K, P, false, 128) || !make_map_gg(&mapB, Wr, K, C, false, prm.N) ||
        !make_map_gg(&mapBh, Wr, K, C, false, prm.N / 2))
        return WG2X2_ERR_LAUNCH;
    return gg_launch<1>(mapA, mapB, prm, st, &mapBh);
}

size_t conv_bwd_tc_workspace_bytes(long long P, int C, int K, int want_dW)
{
    return bwd_ws_layout(P, C, K, want_dW ? conv_dw_tc_splits(P, C, K) : 1).total;
}

// dV and/or dW of the product op on the tensor cores.  V is only needed for dW and for the ReLU mask.
int conv_bwd_tc(const float *V, const float *Wt, const float *dY, const float *mask, float *dV, float *dW, int B, int H, int W,
                int C, int K, int layout, int relu, void *ws, size_t ws_bytes, cudaStream_t st)
{
    if (!tc_bwd_shape_supported(C, K)) return WG2X2_ERR_UNSUPPORTED;
    // TMA bases and the 16-byte loads/stores of the producer and the epilogues: every operand that is given
    // must sit on a 16-byte boundary (checked before anything is enqueued)
    if (misaligned16(V) || misaligned16(Wt) || misaligned16(dY) || misaligned16(mask) || misaligned16(dV) || misaligned16(dW))
        return WG2X2_ERR_BAD_ARG;
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const long long P = (long long)B * nH * nW;
    const int splits = dW ? conv_dw_tc_splits(P, C, K) : 1;
    const BwdWs lay = bwd_ws_layout(P, C, K, splits);
    if (!ws || ws_bytes < lay.total || (reinterpret_cast<uintptr_t>(ws) & 255u)) return WG2X2_ERR_WORKSPACE;
    char *wsb = static_cast<char *>(ws);
    float *dM = reinterpret_cast<float *>(wsb + lay.dm);
    int s = launch_dm(dY, dM, B, H, W, K, layout, st);
    if (s != WG2X2_OK) return s;
    if (dV) {
        s = conv_dv_tc(V, Wt, dM, reinterpret_cast<float *>(wsb + lay.wr), reinterpret_cast<unsigned long long *>(wsb + lay.map), dV,
                       P, C, K, relu, st);
        if (s != WG2X2_OK) return s;
    }
    if (dW) {
        s = conv_dw_tc(V, dM, mask, dW, reinterpret_cast<float *>(wsb + lay.partial), P, C, K, st);
        if (s != WG2X2_OK) return s;
    }
    return WG2X2_OK;
}

// ---------------------------------------------------------------------------------------
// Wide forward path for layers with many channels (C, K >= 256): the 16 products as plain GEMMs with
// N = 256 output channels per unit (conv_grad_gemm_tc_kernel<1>: same operands' major-ness as dV), the
// products M (16, P, K) written once to scratch memory, then one HBM-bound pass for A^T m A.  With N = 64
// (the row-walk kernel, which needs four accumulators live per unit) every A tile is re-read from L2 and
// from shared memory four times as often, and that, not HBM, is what bounds these shapes.
// ---------------------------------------------------------------------------------------
struct OutExtras {
    const float *scale, *shift, *residual;
};

// NHWC: one thread = one tile x 4 output channels
__global__ void __launch_bounds__(256) out_transform_nhwc_kernel(const float *__restrict__ M, float *__restrict__ Y, long long P,
                                                                   int nH, int nW, int K, int outH, int outW, OutExtras ex)
{
    const int KV = K >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P * KV) return;
    const int kv = (int)(idx % KV);
    const long long p = idx / KV;
    const int tw = (int)(p % nW), th = (int)((p / nW) % nH), b = (int)(p / ((long long)nW * nH));
    float4 y[2][2];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) y[a][e] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 m[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) m[j] = __ldg(reinterpret_cast<const float4 *>(M + ((long long)(4 * i + j) * P + p) * K) + kv);
        const float4 z0 = make_float4(m[0].x + m[1].x + m[2].x, m[0].y + m[1].y + m[2].y, m[0].z + m[1].z + m[2].z, m[0].w + m[1].w + m[2].w);
        const float4 z1 = make_float4(m[1].x - m[2].x - m[3].x, m[1].y - m[2].y - m[3].y, m[1].z - m[2].z - m[3].z, m[1].w - m[2].w - m[3].w);
        if (i <= 2) { y[0][0] = y[0][0] + z0; y[0][1] = y[0][1] + z1; }
        if (i == 1) { y[1][0] = y[1][0] + z0; y[1][1] = y[1][1] + z1; }
        if (i >= 2) { y[1][0] = y[1][0] - z0; y[1][1] = y[1][1] - z1; }
    }
    float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ex.scale) { sc = __ldg(reinterpret_cast<const float4 *>(ex.scale) + kv); sh = __ldg(reinterpret_cast<const float4 *>(ex.shift) + kv); }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int h = 2 * th + a, w = 2 * tw + e;
            if (h >= outH || w >= outW) continue;
            const long long o = ((((long long)b * outH + h) * outW + w) * K) / 4 + kv;
            float4 v = y[a][e];
            if (ex.scale) { v.x = fmaf(v.x, sc.x, sh.x); v.y = fmaf(v.y, sc.y, sh.y); v.z = fmaf(v.z, sc.z, sh.z); v.w = fmaf(v.w, sc.w, sh.w); }
            if (ex.residual) { const float4 r = __ldg(reinterpret_cast<const float4 *>(ex.residual) + o); v = v + r; }
            reinterpret_cast<float4 *>(Y)[o] = v;
        }
}

// NCHW: lane = output channel over a band of R tile rows; the 2R x outW pixels of each channel collect in
// shared memory and leave as one contiguous run per channel.
__global__ void __launch_bounds__(256) out_transform_nchw_kernel(const float *__restrict__ M, float *__restrict__ Y, long long P,
                                                                   int nH, int nW, int K, int outH, int outW, int R, int nbands,
                                                                   int pitch, OutExtras ex)
{
    extern __shared__ float O[];
    const int band = blockIdx.x % nbands;
    const int b = blockIdx.x / nbands;
    const int k0 = blockIdx.y * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int th0 = band * R;
    const int rows_blk = min(R, nH - th0);
    const bool k_ok = k0 + lane < K;
    const float sc = (ex.scale && k_ok) ? __ldg(ex.scale + k0 + lane) : 1.f;
    const float sh = (ex.scale && k_ok) ? __ldg(ex.shift + k0 + lane) : 0.f;
    for (int q = warp; q < rows_blk * nW; q += 8) {
        const int br = q / nW, tw = q - br * nW;
        const long long p = ((long long)b * nH + th0 + br) * nW + tw;
        float y[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        if (k_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float m[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) m[j] = __ldg(M + ((long long)(4 * i + j) * P + p) * K + k0 + lane);
                float z0, z1;
                at_cols(m[0], m[1], m[2], m[3], z0, z1);
                at_rows_accum(i, z0, z1, y);
            }
        }
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (2 * tw + e < outW) O[lane * pitch + (2 * br + a) * outW + 2 * tw + e] = fmaf(y[a][e], sc, sh);
    }
    __syncthreads();
    const int lo = 2 * th0, hi = min(2 * th0 + 2 * rows_blk, outH);
    const int n = (hi - lo) * outW;
    for (int kk = warp; kk < 32; kk += 8) {
        if (k0 + kk >= K) break;
        const long long o = (((long long)b * K + k0 + kk) * outH + lo) * outW;
        const float *src = O + kk * pitch;
        if (ex.residual) { for (int i = lane; i < n; i += 32) Y[o + i] = src[i] + __ldg(ex.residual + o + i); }
        else             { for (int i = lane; i < n; i += 32) Y[o + i] = src[i]; }
    }
}

bool conv_fwd_wide_preferred(int C, int K) { return C >= 256 && K >= 256 && C % 4 == 0 && K % 4 == 0; }
size_t conv_fwd_wide_workspace_bytes(long long P, int K) { return align_up((size_t)16 * P * K * sizeof(float), 256); }

int conv_fwd_tc_wide(const float *V, const void *prepared, float *Y, int B, int nH, int nW, int C, int K, int outH, int outW,
                     int layout, const float *out_scale, const float *out_shift, const float *residual, void *ws, size_t ws_bytes,
                     cudaStream_t st)
{
    const long long P = (long long)B * nH * nW;
    if (P > 0x7fffffffLL - 128) return WG2X2_ERR_UNSUPPORTED;
    if (!V || !prepared || !Y) return WG2X2_ERR_BAD_ARG;
    if (misaligned16(V) || misaligned16(prepared) || misaligned16(Y) || misaligned16(out_scale) || misaligned16(out_shift) ||
        misaligned16(residual))
        return WG2X2_ERR_BAD_ARG;
    if (!ws || ws_bytes < conv_fwd_wide_workspace_bytes(P, K) || (reinterpret_cast<uintptr_t>(ws) & 255u)) return WG2X2_ERR_WORKSPACE;
    float *M = static_cast<float *>(ws);
    GgParams prm;
    prm.rows = P; prm.cols = K; prm.contr = C;
    prm.N = gg_cols(K);
    prm.nRB = (int)cdivll(P, 128);
    prm.nCB = cdiv(K, prm.N);
    prm.splits = 1;
    prm.chunks_per_split = cdiv(C, 32);
    prm.units = 16 * prm.nRB * prm.nCB;
    prm.direct = 1;
    prm.out = M;
    prm.mask = nullptr;
    // the zero-block map that weights_prepare built behind the packed weights
    prm.block_map = reinterpret_cast<const unsigned long long *>(static_cast<const unsigned char *>(prepared) +
                                                                 align_up((size_t)16 * K * C * sizeof(float), 256));
    prm.map_mode = 1; prm.map_nkb = cdiv(K, kBlockN); prm.mn4 = 0;
    CUtensorMap mapA, mapB, mapBh;
    if (!make_map_gg(&mapA, V, C, P, false, 128) || !make_map_gg(&mapB, static_cast<const float *>(prepared), C, K, false, prm.N) ||
        !make_map_gg(&mapBh, static_cast<const float *>(prepared), C, K, false, prm.N / 2))
        return WG2X2_ERR_LAUNCH;
    int s = gg_launch<1>(mapA, mapB, prm, st, &mapBh);
    if (s != WG2X2_OK) return s;
    OutExtras ex{out_scale, out_shift, residual};
    if (layout == WG2X2_NHWC) {
        out_transform_nhwc_kernel<<<(unsigned)cdivll(P * (K / 4), 256), 256, 0, st>>>(M, Y, P, nH, nW, K, outH, outW, ex);
    } else {
        int R = 384 / (2 * outW);
        if (R < 1) R = 1;
        if (R > nH) R = nH;
        // a small batch: lower bands, so that the grid still gives every SM a few blocks
        while (R > 1 && (long long)B * cdiv(nH, R) * cdiv(K, 32) < 3LL * kNumSMs) --R;
        const int nbands = cdiv(nH, R);
        R = cdiv(nH, nbands);
        const int pitch = (2 * R * outW) | 1;
        const int smem = 32 * pitch * (int)sizeof(float);
        if ((long long)B * nbands > 0x7fffffffLL || smem > 200 * 1024) return WG2X2_ERR_UNSUPPORTED;
        if (cudaFuncSetAttribute(out_transform_nchw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        out_transform_nchw_kernel<<<dim3((unsigned)(B * nbands), cdiv(K, 32)), 256, smem, st>>>(M, Y, P, nH, nW, K, outH, outW, R,
                                                                                                 nbands, pitch, ex);
    }
    return launch_status();
}
