// Tensor-core gradient products.  Included by conv_tc.cu (same translation unit: the kernels share the
// PTX wrappers, the status word and the plane-mode instantiation of the tcgen05 kernel).
//
//   dM  = A dY A^T           conv_dm_*_kernel: one HBM-bound pass, 16 planes [t][P][K], rounded to TF32
//   dV_t = dM_t . W_t^T      the forward tcgen05 kernel in plane mode (A = dM, B = W as stored: (16,C,K)
//                            is already contraction-contiguous for this product), ReLU mask in the epilogue
//   dW_t = V_t^T . dM_t      conv_dw_tc_kernel below (both operands MN-major), split over P
#pragma once

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

__global__ void __launch_bounds__(256) round_tf32_kernel(const float *__restrict__ src, float *__restrict__ dst, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = round_tf32(__ldg(src + i));
}

static int launch_dm(const float *dY, float *dM, int B, int H, int W, int K, int layout, cudaStream_t st)
{
    const int nH = (H + 1) / 2, nW = (W + 1) / 2;
    const long long P = (long long)B * nH * nW;
    if (layout == WG2X2_NHWC) {
        conv_dm_nhwc_kernel<<<(unsigned)cdivll(P * (K / 4), 256), 256, 0, st>>>(dY, dM, P, nH, nW, H, W, K);
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
// Workspace of the tensor-core backward pass: [dM | W rounded to TF32 | all-ones block masks | dW partials]
// ---------------------------------------------------------------------------------------
struct BwdWs {
    size_t dm, wr, masks, partial, total;
};
static BwdWs bwd_ws_layout(long long P, int C, int K, int dw_splits)
{
    BwdWs w;
    w.dm = 0;
    size_t off = align_up((size_t)16 * P * K * sizeof(float), 256);
    w.wr = off;      off += align_up((size_t)16 * C * K * sizeof(float), 256);
    w.masks = off;   off += align_up((size_t)16 * cdiv(C, kBlockN) * sizeof(unsigned long long), 256);
    w.partial = off; off += dw_splits > 1 ? align_up((size_t)dw_splits * 16 * C * K * sizeof(float), 256) : 0;
    w.total = off;
    return w;
}

bool tc_bwd_shape_supported(int C, int K) { return C % 4 == 0 && K % 4 == 0 && C >= 4 && K >= 4; }

int conv_dv_tc(const float *V, const float *Wt, const float *dM, float *Wr, unsigned long long *masks, float *dV, long long P,
               int C, int K, int relu, cudaStream_t st)
{
    const long long n = (long long)16 * C * K;
    round_tf32_kernel<<<(int)min((long long)kNumSMs * 8, cdivll(n, 256)), 256, 0, st>>>(Wt, Wr, n);
    if (launch_status() != WG2X2_OK) return WG2X2_ERR_LAUNCH;
    if (cudaMemsetAsync(masks, 0xFF, (size_t)16 * cdiv(C, kBlockN) * sizeof(unsigned long long), st) != cudaSuccess)
        return WG2X2_ERR_LAUNCH;
    // A = dM (16, P, K), B = W (16, C, K): contraction over K, C output columns
    return tc_launch(1, WG2X2_NHWC, dM, Wr, masks, dV, relu ? V : nullptr, P, 1, 1, K, C, 0, 0, st);
}

// ---------------------------------------------------------------------------------------
// dW_t[c][k] = sum_p V_t[p][c] dM_t[p][k] on the tensor cores.
//
// Both operands are stored with the contraction index p as the slow axis, i.e. they are "MN-major" for
// UMMA: a [32 p x 32 channel] box lands in shared memory as 32 rows of 128 bytes (128B swizzle, 32B atoms),
// which is one MN block of 32 channels x eight K groups of 4 tiles.  A (V_t^T, M = 128 input channels) is four such
// boxes 4 KB apart (the descriptor's leading-dimension offset), B (dM_t, N = 64/128/256 output channels) is
// N/32 of them.  One MMA (K = 8 tiles) reads 8 rows: start address + 1024 B per step.
// Unit = (position t, 128-channel block of C, N-channel block of K, split of the P range); accumulator in
// TMEM (N columns, double-buffered); the epilogue writes the [128 x N] tile -- dW itself (times the mask)
// when there is one split, else that split's partial sum for conv_dw_reduce_kernel.
// ---------------------------------------------------------------------------------------
constexpr int kDwStages = 4;
constexpr int kDwBoxBytes = 32 * 32 * 4;                 // [32 p][32 ch] fp32
constexpr int kDwABytes = 4 * kDwBoxBytes;               // 128 input channels
constexpr int kDwBBytesMax = 8 * kDwBoxBytes;            // up to 256 output channels
constexpr int kDwStageBytes = kDwABytes + kDwBBytesMax;  // 48 KB
constexpr int kDwSmemBytes = kDwStages * kDwStageBytes + 1024 + kCtrlBytes + kEpiWarps * kEpiStageBytes;

struct DwParams {
    float *out;
    const float *mask;
    long long P;
    int C, K, N;
    int nCB, nKB;
    int splits, chunks_per_split;
    int units;
    int direct;
};

// MN-major TF32 operand.  The only shared-memory layout UMMA accepts for it is the 128-byte swizzle with a
// 32-byte base (layout type 1; TMA writes it with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): rows of 128 bytes,
// the 32-byte chunk index XORed with (row & 3), pattern repeating every 4 rows.  MN blocks of 32 elements
// are 4 KB apart (leading-dimension offset), K groups of 4 rows 512 B apart (stride offset).
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(kDwBoxBytes >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

__global__ void __launch_bounds__(kTcThreads, 1)
conv_dw_tc_kernel(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapM, const DwParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - raw);
    const uint32_t bars = base + kDwStages * kDwStageBytes;
    uint64_t *bars_gen = reinterpret_cast<uint64_t *>(gen_base + kDwStages * kDwStageBytes);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kDwStages + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * kDwStages + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * kDwStages + 2 + b); };
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bars_gen + 2 * kDwStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_gen + 2 * kDwStages + 5);
    float *epi_stage_all = reinterpret_cast<float *>(gen_base + kDwStages * kDwStageBytes + kCtrlBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kDwStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
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
    const uint32_t tmem_base = *tmem_ptr_slot;

    const int N = prm.N;
    const int per_t = prm.nCB * prm.nKB;
    // unit -> (split, t, cb, kb), kb fastest so that neighbouring CTAs share the V tile in L2
    auto decode = [&](int u, int &split, int &t, int &cb, int &kb) {
        kb = u % prm.nKB; u /= prm.nKB;
        cb = u % prm.nCB; u /= prm.nCB;
        t = u % 16;
        split = u / 16;
    };
    (void)per_t;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            const uint32_t stage_tx = (uint32_t)(kDwABytes + (N / 32) * kDwBoxBytes);
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int split, t, cb, kb;
                decode(u, split, t, cb, kb);
                const long long pbeg = (long long)split * prm.chunks_per_split * 32;
                const long long pend = min(prm.P, pbeg + (long long)prm.chunks_per_split * 32);
                for (long long pc = pbeg; pc < pend; pc += 32) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 0x500u | s)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), stage_tx);
                    const uint32_t a_dst = base + s * kDwStageBytes;
                    const uint32_t b_dst = a_dst + kDwABytes;
#pragma unroll
                    for (int mb = 0; mb < 4; ++mb)
                        tma_load_3d(a_dst + mb * kDwBoxBytes, &mapV, full_bar(s), cb * 128 + mb * 32, (int)pc, t);
                    for (int nb = 0; nb < N / 32; ++nb)
                        tma_load_3d(b_dst + nb * kDwBoxBytes, &mapM, full_bar(s), kb * N + nb * 32, (int)pc, t);
                    if (++s == kDwStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(128, N) | (1u << 15) | (1u << 16);   // A and B MN-major
            int s = 0; uint32_t ph = 0;
            uint32_t acc_use[2] = {0, 0};
            int buf = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int split, t, cb, kb;
                decode(u, split, t, cb, kb);
                const long long pbeg = (long long)split * prm.chunks_per_split * 32;
                const long long pend = min(prm.P, pbeg + (long long)prm.chunks_per_split * 32);
                if (!mbar_wait(acce_bar(buf), (acc_use[buf] & 1u) ^ 1u, abort_flag, 0x600u | buf)) { ok = false; break; }
                acc_use[buf]++;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 256);
                uint32_t first = 1;
                for (long long pc = pbeg; pc < pend; pc += 32) {
                    if (!mbar_wait(full_bar(s), ph, abort_flag, 0x700u | s)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * kDwStageBytes;
                    const uint64_t adesc = make_desc_mn_sw128(a_addr);
                    const uint64_t bdesc = make_desc_mn_sw128(a_addr + kDwABytes);
#pragma unroll
                    for (int kg = 0; kg < 4; ++kg) {   // next K group of 8 tiles: 1024 B further
                        umma_tf32(d_tmem, adesc + 64u * kg, bdesc + 64u * kg, idesc, first ? 0u : 1u);
                        first = 0;
                    }
                    umma_commit(empty_bar(s));
                    if (++s == kDwStages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(accf_bar(buf));
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
        const long long plane_elems = (long long)16 * prm.C * prm.K;
        for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
            int split, t, cb, kb;
            decode(u, split, t, cb, kb);
            if (!mbar_wait(accf_bar(buf), acc_use[buf] & 1u, abort_flag, 0x800u | (ew << 4) | buf)) { ok = false; break; }
            acc_use[buf]++;
            tc_fence_after();
            const int c = cb * 128 + q * 32 + lane;
            const long long row_off = (prm.direct ? 0 : (long long)split * plane_elems) + ((long long)t * prm.C + c) * prm.K;
            const int ncol_half = N / 2;
            for (int cc = 0; cc < ncol_half; cc += 32) {
                const int col0 = half * ncol_half + cc;
                const int k = kb * N + col0;
                float r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + col0);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld8(taddr + (uint32_t)(ch * 8), &r[ch * 8]);
                tmem_ld_wait();
                const long long my_off = (c < prm.C && k < prm.K) ? row_off + k : -1;
                if (k + 32 <= prm.K && (prm.K & 3) == 0) {
                    __syncwarp();
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8)
                        *reinterpret_cast<float4 *>(stg + lane * 32 + ((c8 ^ (lane & 7)) << 2)) =
                            make_float4(r[4 * c8], r[4 * c8 + 1], r[4 * c8 + 2], r[4 * c8 + 3]);
                    __syncwarp();
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        const int row = 4 * rr + (lane >> 3), ch = lane & 7;
                        const long long off = __shfl_sync(0xffffffffu, my_off, row);
                        float4 v = *reinterpret_cast<const float4 *>(stg + row * 32 + ((ch ^ (row & 7)) << 2));
                        if (off >= 0) {
                            if (prm.direct && prm.mask) {
                                const float4 mk = __ldg(reinterpret_cast<const float4 *>(prm.mask + off + 4 * ch));
                                v.x *= mk.x; v.y *= mk.y; v.z *= mk.z; v.w *= mk.w;
                            }
                            *reinterpret_cast<float4 *>(prm.out + off + 4 * ch) = v;
                        }
                    }
                } else if (my_off >= 0) {
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        if (k + x >= prm.K) continue;
                        float v = r[x];
                        if (prm.direct && prm.mask) v *= __ldg(prm.mask + my_off + x);
                        prm.out[my_off + x] = v;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(buf));
            buf ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// 3-D map over a (16, P, ch) fp32 tensor, ch contiguous: box = 32 channels x 32 rows, 128-B swizzle with 32-B atoms
static bool make_map_dw(CUtensorMap *map, const float *ptr, int ch, long long rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)ch, (cuuint64_t)rows, 16};
    cuuint64_t strides[2] = {(cuuint64_t)ch * 4, (cuuint64_t)rows * ch * 4};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int dw_tc_cols(int K) { return K > 128 ? 256 : (K > 64 ? 128 : 64); }

// Splits of the P range: enough units for every SM, at least 8 chunks of 32 tiles per split
int conv_dw_tc_splits(long long P, int C, int K)
{
    const long long base_units = (long long)16 * cdiv(C, 128) * cdiv(K, dw_tc_cols(K));
    const long long chunks = cdivll(P, 32);
    long long s = cdivll(kNumSMs, base_units);
    const long long max_s = chunks / 8 > 0 ? chunks / 8 : 1;
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    const long long cps = cdivll(chunks, s);
    return (int)cdivll(chunks, cps);
}

int conv_dw_tc(const float *V, const float *dM, const float *mask, float *dW, float *partial, long long P, int C, int K,
               cudaStream_t st)
{
    DwParams prm;
    prm.P = P; prm.C = C; prm.K = K;
    prm.N = dw_tc_cols(K);
    prm.nCB = cdiv(C, 128);
    prm.nKB = cdiv(K, prm.N);
    prm.splits = conv_dw_tc_splits(P, C, K);
    prm.chunks_per_split = (int)cdivll(cdivll(P, 32), prm.splits);
    prm.units = 16 * prm.nCB * prm.nKB * prm.splits;
    prm.direct = prm.splits == 1;
    prm.out = prm.direct ? dW : partial;
    prm.mask = mask;
    CUtensorMap mapV, mapM;
    if (!make_map_dw(&mapV, V, C, P) || !make_map_dw(&mapM, dM, K, P)) return WG2X2_ERR_LAUNCH;
    if (cudaFuncSetAttribute(conv_dw_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDwSmemBytes) != cudaSuccess)
        return WG2X2_ERR_LAUNCH;
    const int grid = prm.units < kNumSMs ? prm.units : kNumSMs;
    conv_dw_tc_kernel<<<grid, kTcThreads, kDwSmemBytes, st>>>(mapV, mapM, prm);
    if (launch_status() != WG2X2_OK) return WG2X2_ERR_LAUNCH;
    if (!prm.direct) {
        const long long n = (long long)16 * C * K;
        dw_reduce_launch(partial, mask, dW, n, prm.splits, st);
    }
    return launch_status();
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
        s = conv_dv_tc(V, Wt, dM, reinterpret_cast<float *>(wsb + lay.wr), reinterpret_cast<unsigned long long *>(wsb + lay.masks),
                       dV, P, C, K, relu, st);
        if (s != WG2X2_OK) return s;
    }
    if (dW) {
        s = conv_dw_tc(V, dM, mask, dW, reinterpret_cast<float *>(wsb + lay.partial), P, C, K, st);
        if (s != WG2X2_OK) return s;
    }
    return WG2X2_OK;
}
