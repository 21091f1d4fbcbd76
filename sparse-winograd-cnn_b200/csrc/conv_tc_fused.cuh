// Fused Winograd-ReLU layer forward, X -> Y in one kernel (NCHW in and out): the transformed input V never
// goes to memory.  Included by conv_tc.cu.
//
// Same row walk as conv_fwd_tc_kernel (four 128x64 accumulators per Winograd row, double-buffered in TMEM,
// A^T m A in the epilogue), but the A operand of every MMA is produced on the SM:
//   * the X producer (warp 0) brings, by TMA, the input rows one Winograd row of a block of tiles needs, for
//     16 channels at a time, into one of three shared-memory buffers; out-of-image rows and columns arrive as
//     zeros, which is the layer's padding;
//   * sixteen transform warps (one thread = one tile x 4 channels) read their 2 x 4 pixels per channel from
//     that buffer, form the four values of Winograd row i of B^T d B, apply the ReLU, round to TF32 and write
//     them into the four [128 x 16] A tiles of the stage ring in the 64-byte-swizzled K-major layout UMMA
//     reads (the transform is bound by instruction issue, hence the many warps);
//   * the W producer (warp 2) brings the matching [64 x 16] weight tiles by TMA;
//   * the MMA issuer (warp 1) and the eight epilogue warps work as in the unfused kernel.
// A unit is NB images x TH tile rows x TW tile columns (at most 128 tiles, one TMEM lane each) x 64 output
// channels.  Each input row is fetched once per Winograd row that uses it (from L2 after the first time);
// HBM sees X once and Y once.
#pragma once

constexpr int kFuStages = 8;                       // two groups of four (one per Winograd column j)
constexpr int kFuABytes = 128 * 64;                // [128 tiles][16 channels] fp32
constexpr int kFuBBytes = 64 * 64;                 // [64 out-channels][16 channels]
constexpr int kFuStageBytes = kFuABytes + kFuBBytes;
constexpr int kFuXbufs = 3;
constexpr int kFuXbufBytes = 40960;
constexpr int kFuXfWarps = 16;                     // transform warps: one thread = one tile x 4 channels of a group
constexpr int kFuThreads = 128 + 256 + 32 * kFuXfWarps;   // control WG, 2 epilogue WGs, 4 transform WGs
constexpr int kFuSmemBytes = kFuStages * kFuStageBytes + kFuXbufs * kFuXbufBytes + kCtrlBytes + 1024;

struct FuParams {
    float *Y;
    const float *out_scale, *out_shift, *residual;
    int B, H, W, C, K, nH, nW, outH, outW;
    int TH, TW, NB, BH, BW;          // block of tiles and the input box that feeds one Winograd row of it
    int nRB, nSeg, nGroups, nKB, nC16;
    int units, relu;
    uint32_t xbytes;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// K-major operand with rows of 64 bytes, 64-byte swizzle: 8-row groups 512 B apart
__device__ __forceinline__ uint64_t make_desc_k_sw64(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;                 // SWIZZLE_64B
    return d;
}

template <bool EXTRAS>
__global__ void __launch_bounds__(kFuThreads, 1)
layer_fwd_fused_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW, const FuParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - raw);
    const uint32_t xbase = base + kFuStages * kFuStageBytes;
    const float *xgen = reinterpret_cast<const float *>(gen_base + kFuStages * kFuStageBytes);
    const uint32_t bars = xbase + kFuXbufs * kFuXbufBytes;
    uint64_t *bars_gen = reinterpret_cast<uint64_t *>(gen_base + kFuStages * kFuStageBytes + kFuXbufs * kFuXbufBytes);
    // barriers: full[8], empty[8], acc_full[2], acc_empty[2], xfull[3], xempty[3]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kFuStages + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * kFuStages + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * kFuStages + 2 + b); };
    auto xfull_bar = [&](int b) { return bars + 8u * (2 * kFuStages + 4 + b); };
    auto xempty_bar = [&](int b) { return bars + 8u * (2 * kFuStages + 4 + kFuXbufs + b); };
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bars_gen + 2 * kFuStages + 4 + 2 * kFuXbufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_gen + 2 * kFuStages + 5 + 2 * kFuXbufs);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kFuStages; ++s) { mbar_init(full_bar(s), 1 + kFuXfWarps); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), kEpiWarps); }
        for (int b = 0; b < kFuXbufs; ++b) { mbar_init(xfull_bar(b), 1); mbar_init(xempty_bar(b), kFuXfWarps); }
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

    const int nC16 = prm.nC16;
    auto decode = [&](int u, int &g, int &rb, int &seg, int &kb) {
        kb = u % prm.nKB; u /= prm.nKB;
        seg = u % prm.nSeg; u /= prm.nSeg;
        rb = u % prm.nRB;
        g = u / prm.nRB;
    };

    // registers: 896 threads x 72 at launch; control warps keep 24, transform warps 40, epilogue warps take 160
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
        if (warp == 0 && lane == 0) {
            // ------------------------------ X producer -----------------------------------
            int xb = 0; uint32_t xph = 0;
            bool ok = true;
            int trx = 0; (void)trx;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int g, rb, seg, kb;
                decode(u, g, rb, seg, kb);
                const int x0 = 2 * seg * prm.TW - 4, th0 = rb * prm.TH, b0 = g * prm.NB;
                for (int i = 0; i < 4 && ok; ++i) {
                    const int h_lo = 2 * th0 - (i == 0 ? 1 : 0);
                    for (int cc = 0; cc < nC16; ++cc) {
                        if (!mbar_wait(xempty_bar(xb), xph ^ 1u, abort_flag, 0x900u | xb)) { ok = false; break; }
                        TC_TRACE(trx); ++trx;
                        mbar_expect_tx(xfull_bar(xb), prm.xbytes);
                        tma_load_4d(xbase + xb * kFuXbufBytes, &mapX, xfull_bar(xb), x0, h_lo, cc * 16, b0);
                        if (++xb == kFuXbufs) { xb = 0; xph ^= 1u; }
                    }
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        } else if (warp == 2 && lane == 0) {
            // ------------------------------ W producer -----------------------------------
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int g, rb, seg, kb;
                decode(u, g, rb, seg, kb);
                for (int i = 0; i < 4 && ok; ++i)
                    for (int cc = 0; cc < nC16 && ok; ++cc)
                        for (int j = 0; j < 4; ++j) {
                            if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 0xA00u | s)) { ok = false; break; }
                            mbar_expect_tx(full_bar(s), kFuBBytes);
                            tma_load_3d(base + s * kFuStageBytes + kFuABytes, &mapW, full_bar(s), cc * 16, kb * kBlockN, 4 * i + j);
                            if (++s == kFuStages) { s = 0; ph ^= 1u; }
                        }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        } else if (warp == 1 && lane == 0) {
            // ------------------------------ MMA issuer -----------------------------------
            constexpr uint32_t idesc = make_idesc_tf32(kBlockM, kBlockN);
            int s = 0; uint32_t ph = 0;
            uint32_t acc_use[2] = {0, 0};
            bool ok = true;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                for (int i = 0; i < 4 && ok; ++i) {
                    const int buf = i & 1;
                    if (!mbar_wait(acce_bar(buf), (acc_use[buf] & 1u) ^ 1u, abort_flag, 0x200u | buf)) { ok = false; break; }
                    acc_use[buf]++;
                    tc_fence_after();
                    for (int cc = 0; cc < nC16 && ok; ++cc)
                        for (int j = 0; j < 4; ++j) {
                            if (!mbar_wait(full_bar(s), ph, abort_flag, 0x300u | s)) { ok = false; break; }
                            tc_fence_after();
                            const uint32_t a_addr = base + s * kFuStageBytes;
                            const uint64_t adesc = make_desc_k_sw64(a_addr);
                            const uint64_t bdesc = make_desc_k_sw64(a_addr + kFuABytes);
                            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 4 * kBlockN + j * kBlockN);
#pragma unroll
                            for (int kk = 0; kk < 2; ++kk)
                                umma_tf32(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (cc > 0 || kk > 0) ? 1u : 0u);
                            umma_commit(empty_bar(s));
                            if (++s == kFuStages) { s = 0; ph ^= 1u; }
                        }
                    if (ok) umma_commit(accf_bar(buf));
                }
            }
        }
    } else if (warp >= 12) {
        // ------------------------------ transform warps ----------------------------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        const int l = ((warp - 12) & 3) * 32 + lane;           // tile = TMEM lane = A-tile row
        const int c4 = (warp - 12) >> 2;                       // which 4 of the group's 16 channels
        const int per_img = prm.TH * prm.TW;
        const bool live = l < prm.NB * per_img;
        const int le = live ? l : 0;                            // dead lanes (block smaller than 128 tiles) shadow tile 0:
        const int bi = le / per_img, rem = le - bi * per_img;   // their A rows feed TMEM lanes nobody reads
        const int thl = rem / prm.TW, twl = rem - thl * prm.TW;
        const bool edge_l = (lane == 0) || (twl == 0) || !live;
        const bool edge_r = (lane == 31) || (twl == prm.TW - 1) || !live;
        const int BH = prm.BH, BW = prm.BW;
        const uint32_t swz = (uint32_t)((l >> 1) & 3);
        int xb = 0; uint32_t xph = 0;
        int s = 0; uint32_t ph = 0;
        bool ok = true;
        int trt = 0; (void)trt;
        for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
            for (int i = 0; i < 4 && ok; ++i) {
                const int rowA = 2 * thl, rowB = 2 * thl + ((i == 0 || i == 3) ? 2 : 1);
                for (int cc = 0; cc < nC16; ++cc) {
                    if (warp == 12 && lane == 0) TC_TRACE(512 + 4 * trt);
                    if (!mbar_wait(xfull_bar(xb), xph, abort_flag, 0xB00u | xb)) { ok = false; break; }
                    if (warp == 12 && lane == 0) TC_TRACE(512 + 4 * trt + 1);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (ok && !mbar_wait(empty_bar(s + j), ph ^ 1u, abort_flag, 0xC00u | (s + j))) ok = false;
                    if (!ok) break;
                    if (warp == 12 && lane == 0) TC_TRACE(512 + 4 * trt + 2);
                    const float *xb_ptr = xgen + xb * (kFuXbufBytes / 4) + (bi * 16 * BH) * BW + 2 * twl + 3;
                    uint8_t *a_tiles = gen_base + s * kFuStageBytes + l * 64;
                    {
                        float o[4][4];   // [j][channel within the quad]
#pragma unroll
                        for (int cq = 0; cq < 4; ++cq) {
                            // each lane reads the two pixels its tile owns as one 8-byte load per row and takes the
                            // two halo pixels from its neighbours' registers; only lanes at the edge of a tile row
                            // (or of the warp) read them from shared memory
                            const float *pa = xb_ptr + ((c4 * 4 + cq) * BH + rowA) * BW;
                            const float *pb = xb_ptr + ((c4 * 4 + cq) * BH + rowB) * BW;
                            const float2 am = *reinterpret_cast<const float2 *>(pa + 1);
                            const float2 bm = *reinterpret_cast<const float2 *>(pb + 1);
                            float a0 = __shfl_up_sync(0xffffffffu, am.y, 1), a3 = __shfl_down_sync(0xffffffffu, am.x, 1);
                            float b0 = __shfl_up_sync(0xffffffffu, bm.y, 1), b3 = __shfl_down_sync(0xffffffffu, bm.x, 1);
                            if (edge_l) { a0 = pa[0]; b0 = pb[0]; }
                            if (edge_r) { a3 = pa[3]; b3 = pb[3]; }
                            float r[4];
                            if (i == 1)      { r[0] = a0 + b0; r[1] = am.x + bm.x; r[2] = am.y + bm.y; r[3] = a3 + b3; }
                            else if (i == 2) { r[0] = b0 - a0; r[1] = bm.x - am.x; r[2] = bm.y - am.y; r[3] = b3 - a3; }
                            else             { r[0] = a0 - b0; r[1] = am.x - bm.x; r[2] = am.y - bm.y; r[3] = a3 - b3; }
                            float v0 = r[0] - r[2], v1 = r[1] + r[2], v2 = r[2] - r[1], v3 = r[1] - r[3];
                            if (prm.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
                            // stored as fp32: the tensor core reads the upper 19 bits (TF32), as it does for V from memory
                            o[0][cq] = v0; o[1][cq] = v1; o[2][cq] = v2; o[3][cq] = v3;
                        }
                        const uint32_t chunk = ((uint32_t)c4 ^ swz) << 4;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<float4 *>(a_tiles + j * kFuStageBytes + chunk) = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
                    }
                    // make the generic-proxy writes visible to the tensor core's async proxy, then publish
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (warp == 12 && lane == 0) TC_TRACE(512 + 4 * trt + 3);
                    ++trt;
                    if (lane == 0) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) mbar_arrive(full_bar(s + j));
                        mbar_arrive(xempty_bar(xb));
                    }
                    s += 4;
                    if (s == kFuStages) { s = 0; ph ^= 1u; }
                    if (++xb == kFuXbufs) { xb = 0; xph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
        const int ew = warp - 4;
        const int q = warp & 3;
        const int half = ew >> 2;
        const int l = q * 32 + lane;
        const int per_img = prm.TH * prm.TW;
        const int bi = l / per_img, rem = l - bi * per_img;
        const int thl = rem / prm.TW, twl = rem - thl * prm.TW;
        uint32_t acc_use[2] = {0, 0};
        bool ok = true;
        for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
            int g, rb, seg, kb;
            decode(u, g, rb, seg, kb);
            float y[4][32];
#pragma unroll
            for (int o = 0; o < 4; ++o)
#pragma unroll
                for (int c = 0; c < 32; ++c) y[o][c] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int buf = i & 1;
                if (ok && !mbar_wait(accf_bar(buf), acc_use[buf] & 1u, abort_flag, 0x400u | (ew << 4) | buf)) ok = false;
                acc_use[buf]++;
                if (ok) {
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 4 * kBlockN + half * 32);
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        float m[4][8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) tmem_ld8(taddr + (uint32_t)(j * kBlockN + ch * 8), m[j]);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            float z0, z1;
                            at_cols(m[0][c], m[1][c], m[2][c], m[3][c], z0, z1);
                            if (i <= 2) { y[0][ch * 8 + c] += z0; y[1][ch * 8 + c] += z1; }
                            if (i == 1) { y[2][ch * 8 + c] += z0; y[3][ch * 8 + c] += z1; }
                            if (i >= 2) { y[2][ch * 8 + c] -= z0; y[3][ch * 8 + c] -= z1; }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acce_bar(buf));
                }
            }
            if (!ok) break;
            const int b = g * prm.NB + bi, th = rb * prm.TH + thl, tw = seg * prm.TW + twl;
            const bool tile_ok = (l < prm.NB * per_img) && b < prm.B && th < prm.nH && tw < prm.nW;
            const int kbase = kb * kBlockN + half * 32;
            if (tile_ok) {
                const bool pair = (prm.outW & 1) == 0;
                const long long cstride = (long long)prm.outH * prm.outW;
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const int h = 2 * th + a;
                    if (h >= prm.outH) continue;
                    const long long o0 = (((long long)b * prm.K + kbase) * prm.outH + h) * prm.outW + 2 * tw;
#pragma unroll
                    for (int cg = 0; cg < 32; cg += 8) {
                        float2 rs[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            rs[c] = make_float2(0.f, 0.f);
                            if (EXTRAS && prm.residual && kbase + cg + c < prm.K) {
                                const float *rp = prm.residual + o0 + (cg + c) * cstride;
                                if (pair) rs[c] = __ldg(reinterpret_cast<const float2 *>(rp));
                                else { rs[c].x = __ldg(rp); if (2 * tw + 1 < prm.outW) rs[c].y = __ldg(rp + 1); }
                            }
                        }
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            if (kbase + cg + c >= prm.K) continue;
                            float v0 = y[2 * a][cg + c], v1 = y[2 * a + 1][cg + c];
                            if (EXTRAS && prm.out_scale) {
                                const float s1 = __ldg(prm.out_scale + kbase + cg + c), b1 = __ldg(prm.out_shift + kbase + cg + c);
                                v0 = fmaf(v0, s1, b1); v1 = fmaf(v1, s1, b1);
                            }
                            if (EXTRAS) { v0 += rs[c].x; v1 += rs[c].y; }
                            float *dst = prm.Y + o0 + (cg + c) * cstride;
                            if (pair) *reinterpret_cast<float2 *>(dst) = make_float2(v0, v1);
                            else { dst[0] = v0; if (2 * tw + 1 < prm.outW) dst[1] = v1; }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
// Shapes the fused kernel takes: NCHW, row length a multiple of 4 floats (TMA strides are multiples of
// 16 bytes), channels a multiple of 16.
bool fused_fwd_supported(int B, int H, int W, int C, int K, int layout)
{
    (void)B; (void)H; (void)K;
    return layout == WG2X2_NCHW && (W % 4 == 0) && (C % 16 == 0) && C >= 16;
}

static bool fused_geometry(FuParams &p)
{
    p.nH = (p.H + 1) / 2; p.nW = (p.W + 1) / 2;
    p.TW = p.nW <= 32 ? p.nW : 32;
    p.nSeg = cdiv(p.nW, p.TW);
    p.BW = (2 * p.TW + 5 + 3) & ~3;
    int TH = kBlockM / p.TW;
    if (TH > p.nH) TH = p.nH;
    while (TH > 1 && (size_t)p.BW * (2 * TH + 1) * 16 * 4 > (size_t)kFuXbufBytes) --TH;
    if ((size_t)p.BW * (2 * TH + 1) * 16 * 4 > (size_t)kFuXbufBytes) return false;
    p.TH = TH;
    p.BH = 2 * TH + 1;
    p.NB = 1;
    if (TH == p.nH) {
        int nb = kBlockM / (TH * p.TW);
        while (nb > 1 && (size_t)p.BW * p.BH * 16 * 4 * nb > (size_t)kFuXbufBytes) --nb;
        if (nb > p.B) nb = p.B;
        p.NB = nb < 1 ? 1 : nb;
    }
    p.nRB = cdiv(p.nH, p.TH);
    p.nGroups = cdiv(p.B, p.NB);
    p.nKB = cdiv(p.K, kBlockN);
    p.nC16 = p.C / 16;
    p.xbytes = (uint32_t)((size_t)p.BW * p.BH * 16 * p.NB * 4);
    const long long units = (long long)p.nGroups * p.nRB * p.nSeg * p.nKB;
    if (units > 0x7fffffffLL) return false;
    p.units = (int)units;
    return true;
}

int layer_fwd_fused(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                    const float *out_scale, const float *out_shift, const float *residual, cudaStream_t st)
{
    if (!X || !prepared || !Y) return WG2X2_ERR_BAD_ARG;
    if (!fused_fwd_supported(B, H, W, C, K, WG2X2_NCHW)) return WG2X2_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (reinterpret_cast<uintptr_t>(Y) & 7u)) return WG2X2_ERR_BAD_ARG;
    if ((out_scale == nullptr) != (out_shift == nullptr)) return WG2X2_ERR_BAD_ARG;
    FuParams p;
    p.Y = Y; p.out_scale = out_scale; p.out_shift = out_shift; p.residual = residual;
    p.B = B; p.H = H; p.W = W; p.C = C; p.K = K; p.outH = H; p.outW = W; p.relu = relu;
    if (!fused_geometry(p)) return WG2X2_ERR_UNSUPPORTED;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return WG2X2_ERR_LAUNCH;
    CUtensorMap mapX, mapW;
    {
        cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)B};
        cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4, (cuuint64_t)C * H * W * 4};
        cuuint32_t box[4] = {(cuuint32_t)p.BW, (cuuint32_t)p.BH, 16, (cuuint32_t)p.NB};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (fn(&mapX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(X), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)K, 16};
        cuuint64_t strides[2] = {(cuuint64_t)C * 4, (cuuint64_t)K * C * 4};
        cuuint32_t box[3] = {16, (cuuint32_t)kBlockN, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (fn(&mapW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(prepared), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
    }
    // a grid that divides the units evenly: every CTA runs the same number of them
    const int rounds = cdiv(p.units, kNumSMs);
    const int grid = cdiv(p.units, rounds);
    const bool extras = out_scale || residual;
    if (extras) {
        if (cudaFuncSetAttribute(layer_fwd_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFuSmemBytes) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        layer_fwd_fused_kernel<true><<<grid, kFuThreads, kFuSmemBytes, st>>>(mapX, mapW, p);
    } else {
        if (cudaFuncSetAttribute(layer_fwd_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFuSmemBytes) != cudaSuccess)
            return WG2X2_ERR_LAUNCH;
        layer_fwd_fused_kernel<false><<<grid, kFuThreads, kFuSmemBytes, st>>>(mapX, mapW, p);
    }
    return launch_status();
}
