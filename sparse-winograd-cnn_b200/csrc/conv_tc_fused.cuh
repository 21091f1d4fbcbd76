// Fused Winograd-ReLU layer forward, X -> Y in one kernel (NCHW in and out): neither the transformed input V
// nor the 16 Winograd-domain products ever exist outside the SM.  Included by conv_tc.cu.
//
// Both transforms ride on the tensor core's operands:
//   * input side: the A operand of every MMA (position (i, j) of B^T d B for 128 tiles x 8 channels, after
//     the ReLU) is computed by the transform warps and written with tcgen05.st into tensor memory
//     (lane = tile, column = channel); tcgen05.mma reads it from there;
//   * output side: y[a][e] = sum_ij At[a][i] At[e][j] (V_ij . W_ij) is linear in the products and the
//     coefficients are 0 / +1 / -1, so position (i, j) is accumulated straight into the (up to four) output
//     accumulators (a, e) it contributes to, with the instruction descriptor's negate bit for the minus
//     signs.  That costs 36 instead of 16 MMAs per 8 channels (the tensor core has the room) and leaves four
//     128x64 accumulators per unit instead of sixteen products: the epilogue only copies.
// A unit walks the Winograd rows in three phases, so that output row a = 0 is complete (and drains) before the
// last phase and a = 1 drains under the next unit's first:
//   phase A  row i = 0            slots of 32 input channels: four [128 x 32] A tiles + four [64 x 32] weight tiles
//   phase B  rows i = 1 and 2     slots of 16 input channels: eight [128 x 16] A tiles + eight [64 x 16] weight tiles;
//                                 both rows are built from the same two input rows (d1 + d2 and d2 - d1), which
//                                 therefore travel to shared memory and to the registers once for the two of them
//   phase C  row i = 3            as phase A
// Every slot is one A group of 128 tensor-memory columns and 32 KB of weights, and carries 48 MMAs (24 in the
// phases where only one output row takes part).  A step is one team's half of a slot:
//   * the X producer (warp 4) brings, by TMA, the input rows a step needs into a ring of shared-memory
//     buffers: rows d0,d2 (phase A) or d1,d3 (phase C) of 16 channels through a tensor map that walks the image
//     with a row stride of 2, rows d1,d2 of 8 channels as a dense box in phase B; out-of-image rows, columns and
//     channels arrive as zeros, which is the layer's padding;
//   * two teams of eight transform warps fill the two halves of every slot side by side; a thread owns one
//     tile: two 8-byte loads per channel give the middle pixels of its window, the outer two come from the
//     neighbouring lanes by shuffle; an optional per-channel affine map (a BatchNorm in front of the layer) is
//     applied on the fly without touching the zero padding;
//   * the W producer (warp 6) streams the slot's weight tiles (B operands);
//   * four MMA issuers (warps 0..3), one per output accumulator (a, e): each walks its loop as a whole warp with
//     warp-uniform operands and lets one elected lane issue (a lone lane issuing from per-thread registers takes
//     several times as many issue slots, for which the transform warps compete);
//   * the eight epilogue warps read output row a = 0 as soon as phase B is done and row a = 1 after phase C, stage
//     16 channels at a time in one of two shared-memory boxes (optional per-channel affine) and hand the box to a
//     TMA store (row stride 2 in Y), which also clips odd sizes and partial blocks -- or to a TMA reduce-add when
//     Y already holds a shortcut to add to.
// Tensor memory: columns 0..255 = the accumulators (a, e) at (2a + e) * 64, 256..511 = a ring of two A groups.
// A unit is NB images x TH tile rows x TW tile columns (at most 128 tiles, one TMEM lane each; a tile row takes
// a power-of-two number of lanes) x 64 output channels.  HBM sees X once and Y once.
// Every waiter sees every phase of a barrier it waits on (a parity wait cannot tell a phase from the one two
// before it); all waits are bounded and end in a status word instead of a hang.
#pragma once
#include <type_traits>

constexpr int kFuAGroups = 2;                      // ring of A groups in tensor memory; a group = four [128 x 32] tiles
constexpr int kFuGroupCols = 4 * 32;               // tensor-memory columns of an A group (phase B: 8 tiles x 16)
constexpr int kFuACol0 = 4 * kBlockN;              // first tensor-memory column of the A ring
constexpr int kFuWStages = kFuAGroups;            // a W stage travels with its A group: one "slot" of the ring
constexpr int kFuWTile = 64 * 128;                 // one [64 out-channels][32 channels] tile, rows of 128 bytes
constexpr int kFuWBytes = 4 * kFuWTile;            // four of them, one per Winograd column j
#ifndef WG_FU_XBUFS
#define WG_FU_XBUFS 5
#endif
#ifndef WG_FU_YBOXES
#define WG_FU_YBOXES 1
#endif
constexpr int kFuXbufs = WG_FU_XBUFS;
constexpr int kFuXfull = 2 * kFuXbufs;             // full-barriers of the X ring (see the kernel)
constexpr int kFuXbufBytes = 24576;                // the larger box: (TH + 1) rows x BW x 16 channels x NB images
constexpr int kFuYBoxes = WG_FU_YBOXES;            // staging boxes of Y per epilogue warpgroup
constexpr int kFuTeamWarps = 8;                    // transform warps per team: one thread = one tile x 8 channels
constexpr int kFuThreads = 256 + 256 + 2 * 32 * kFuTeamWarps;   // 2 control WGs, 2 epilogue WGs, 2 transform teams (2 WGs each)
constexpr int kFuYStageBytes = 16384;              // one [NB][16 channels][TH rows][2*TW pixels] box of Y
constexpr int kFuW2Tile = 64 * 64;                 // phase B: one [64 out-channels][16 channels] tile, rows of 64 bytes
constexpr int kFuSmemBytes = kFuWStages * kFuWBytes + kFuXbufs * kFuXbufBytes + 2 * kFuYBoxes * kFuYStageBytes + kCtrlBytes + 1024;
static_assert(kFuACol0 + kFuAGroups * kFuGroupCols <= (int)kTmemCols, "tensor memory columns");
static_assert(kFuSmemBytes <= 232448, "shared memory per CTA");
// Register hand-over (setmaxnreg): the kernel starts with 64 registers per thread; the increase of the transform
// warps can only be served from what the other warps of the same CTA have given back, and it blocks (for
// ever) if that is not enough, so the three shares must fit into the launch allocation.
constexpr int kFuRegsLaunch = 64, kFuRegsCtrl = 32, kFuRegsXf = 80, kFuRegsEpi = 64;
static_assert(256 * kFuRegsCtrl + 256 * kFuRegsEpi + 2 * 32 * kFuTeamWarps * kFuRegsXf <= kFuRegsLaunch * kFuThreads,
              "setmaxnreg shares exceed the registers the CTA was launched with");

#ifdef WG_TC_TRACE   // development aid: wall-clock stamps (ns) of every CTA at entry, after set-up and at its end
#define FU_CTA_STAMP(k) do { if (threadIdx.x == 0 && blockIdx.x < 200) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_tc_trace[3200 + 4 * blockIdx.x + (k)] = (long long)t_; } } while (0)
#else
#define FU_CTA_STAMP(k) do { } while (0)
#endif

struct FuParams {
    float *Y;
    const float *out_scale, *out_shift;
    int accumulate;                        // Y already holds the shortcut: add to it (TMA reduce) instead of overwriting
    const float *in_scale, *in_shift;      // per input channel, applied to the image before the transform (AFFINE)
    const unsigned long long *masks;       // zero-block map of the prepared weights: bit cc of masks[t][kb]
    int B, H, W, C, K, nH, nW, outH, outW;
    int TH, TW, NB, BW, BWY;         // block of tiles; BW = width of the input box, BWY = of the output box
    int lp_log2;                     // a tile row takes 2^lp_log2 >= TW TMEM lanes
    int nRB, nSeg, nGroups, nKB, nC32;        // nC32 = ring slots (32 input channels each) per Winograd row
    int units, relu;
    uint32_t xbytes1, xbytes2;       // bytes of the dense (2*TH rows, 8 channels) and of the row-stride-2 (TH+1 rows, 16 channels) box
    uint32_t spin_limit;             // polls before a wait gives up (wg2x2_set_wait_limit)
    int drop_load;                   // >= 0: the W producer of CTA 0 leaves out its drop_load-th slot (wg2x2_test_drop_load), else -1
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// Bounded wait for roles that can afford a late wake-up: sleeps between polls, so that the waiting warp leaves
// the issue slots of its scheduler to the warps that have work.
__device__ __forceinline__ bool mbar_wait_sleepy(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned where, unsigned ns,
                                                 uint32_t limit = kSpinLimit)
{
    for (uint32_t it = 0; it < limit / 8 + 1; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(ns);
        if ((it & 255) == 255 && *abort_flag) { g_tc_diag[(where >> 8) & 31] = where | (parity << 16) | 0x40000000u; return false; }
    }
    *abort_flag = 1;
    g_tc_diag[(where >> 8) & 31] = where | (parity << 16) | 0x80000000u;
    g_tc_status[1] = where;
    g_tc_status[0] = 1;
    return false;
}

// shared memory -> global, clipped to the tensor; completion is tracked by the thread's bulk async-groups
__device__ __forceinline__ void tma_store_4d(uint32_t src, const CUtensorMap *map, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%1, {%2, %3, %4, %5}], [%0];"
        ::"r"(src), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// the same box added to what global memory holds (element-wise fp32 add done by the TMA unit)
__device__ __forceinline__ void tma_reduce_add_4d(uint32_t src, const CUtensorMap *map, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%1, {%2, %3, %4, %5}], [%0];"
        ::"r"(src), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
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

// D[tmem] (+)= A[tmem] * B[smem], M=128, N=kBlockN, K=8 (tf32): A is 128 lanes x 8 columns of tensor memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The two K=8 MMAs of one [128 x 16] A tile: columns a_tmem.. and a_tmem+8.., B descriptors 32 bytes apart.
// The first accumulates only if `accumulate`, the second always.
__device__ __forceinline__ void umma_tf32_ts_x2(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 b0, b1;\n\t.reg .b32 a1, l1;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.eq.b32 q, %4, %4;\n\t"
        "mov.b64 b0, {%2, %3};\n\t"
        "add.u32 l1, %2, 2;\n\t"
        "mov.b64 b1, {l1, %3};\n\t"
        "add.u32 a1, %1, 8;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], b0, %4, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [a1], b1, %4, q;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// 8-byte shared-memory load from a 32-bit shared-space address.  Not volatile: the compiler may schedule it
// freely among the arithmetic; it is kept after the barrier waits by the "memory" clobber of those.
__device__ __forceinline__ float2 lds_f2(uint32_t addr)
{
    float2 v;
    asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}
// 4 registers per thread -> this warp's 32 lanes x 4 consecutive 32-bit columns.
// The tensor core reads the upper 19 bits of each value (TF32) and drops the rest, as it does for V that the
// two-kernel path brings from memory.  Built with -DWG2X2_ROUND_V, half a unit of the last kept place is added to
// the bit pattern first, which turns that truncation into rounding to nearest (magnitude-wise, as cvt.rna.tf32
// does) and removes the one-sided bias of about 2^-12 per product; it costs one integer add per value, measured
// 1.8 % of the kernel's time on the 64 x 64 x 56 x 56 layer, and is off by default.
#ifdef WG2X2_ROUND_V
#define WG_FU_RND(x) (__float_as_uint(x) + 0x1000u)
#else
#define WG_FU_RND(x) __float_as_uint(x)
#endif
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const float *r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                 ::"r"(taddr), "r"(WG_FU_RND(r[0])), "r"(WG_FU_RND(r[1])), "r"(WG_FU_RND(r[2])), "r"(WG_FU_RND(r[3]))
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool EXTRAS, bool AFFINE>
__global__ void __launch_bounds__(kFuThreads, 1)
layer_fwd_fused_kernel(const __grid_constant__ CUtensorMap mapXd, const __grid_constant__ CUtensorMap mapXs,
                       const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapW2,
                       const __grid_constant__ CUtensorMap mapY, const FuParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - raw);
    constexpr int kWOff = 0;
    constexpr int kXOff = kWOff + kFuWStages * kFuWBytes;
    constexpr int kYOff = kXOff + kFuXbufs * kFuXbufBytes;
    constexpr int kBarOff = kYOff + 2 * kFuYBoxes * kFuYStageBytes;
    const uint32_t wbase = base + kWOff, xbase = base + kXOff, bars = base + kBarOff;
    const float *xgen = reinterpret_cast<const float *>(gen_base + kXOff);
    uint64_t *bars_gen = reinterpret_cast<uint64_t *>(gen_base + kBarOff);
    // barriers: full[G] (both halves of the A group written, one by each team, and the W tiles landed), free[G] (the four issuers' MMAs on the
    // slot are complete), acc_full[2] / acc_empty[2] (per output row a), xfull[2*XB], xempty[XB], ywritten[2], yfree[2].
    // Steps 2s and 2s+1 (one per team) fill the two halves of slot s.
    // Step n fills X buffer n % XB but signals xfull[n % (2*XB)]: with an odd XB the two teams take turns on a
    // buffer, and a parity wait can only tell a barrier's current phase from the one before it, so a waiter has
    // to see every phase of the barrier it waits on; xfull[j] is always the same team's.
    constexpr int kB0 = 0, kB1 = kB0 + kFuAGroups, kB4 = kB1 + kFuAGroups,
                  kB5 = kB4 + 2, kB6 = kB5 + 2, kB7 = kB6 + kFuXfull, kB7b = kB7 + kFuXbufs, kB8 = kB7b + 4;
    static_assert((kB8 + 3) <= 32 && (32 + 4 * 16) * 8 <= kCtrlBytes, "control block: barriers, then the issuers' zero-block words");
    auto full_bar = [&](int g) { return bars + 8u * (kB0 + g); };
    auto free_bar = [&](int g) { return bars + 8u * (kB1 + g); };
    auto accf_bar = [&](int b) { return bars + 8u * (kB4 + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (kB5 + b); };
    auto xfull_bar = [&](int b) { return bars + 8u * (kB6 + b); };
    auto xempty_bar = [&](int b) { return bars + 8u * (kB7 + b); };
    auto ywritten_bar = [&](int h) { return bars + 8u * (kB7b + h); };
    auto yfree_bar = [&](int h) { return bars + 8u * (kB7b + 2 + h); };
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bars_gen + kB8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_gen + kB8 + 1);

    // (broadcast from lane 0: the compiler then treats the warp index, and all that is derived from it, as warp-uniform)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    FU_CTA_STAMP(0);

    if (threadIdx.x == 0) {
        for (int g = 0; g < kFuAGroups; ++g) { mbar_init(full_bar(g), 2 * kFuTeamWarps + 1); mbar_init(free_bar(g), 4); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 2); mbar_init(acce_bar(b), kEpiWarps); }
        for (int b = 0; b < kFuXfull; ++b) mbar_init(xfull_bar(b), 1);
        for (int b = 0; b < kFuXbufs; ++b) mbar_init(xempty_bar(b), kFuTeamWarps);
        for (int h = 0; h < 2; ++h) { mbar_init(ywritten_bar(h), 4); mbar_init(yfree_bar(h), 1); }
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
    FU_CTA_STAMP(1);
    // Launched with programmatic stream serialisation, this grid may have been scheduled while the kernel before it in
    // the stream was still running (on SMs that one left free, or as its CTAs ended): everything up to here touched
    // no global memory.  Let the next launch do the same, then wait for the previous grid to have completed and its
    // writes to be visible.  (Both instructions do nothing in a launch without the attribute.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int nC32 = prm.nC32;
    // per unit: slots 0 .. nC32-1 are phase A, nC32 .. 3*nC32-1 phase B, 3*nC32 .. 4*nC32-1 phase C; two steps per slot
    const int spu_slots = 4 * nC32;
    auto decode = [&](int u, int &g, int &rb, int &seg, int &kb) {
        kb = u % prm.nKB; u /= prm.nKB;
        seg = u % prm.nSeg; u /= prm.nSeg;
        rb = u % prm.nRB;
        g = u / prm.nRB;
    };

    // registers: 1024 threads x 64 at launch; control warps keep 32, epilogue warps stay at 64, transform warps take 80
    if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kFuRegsCtrl));
        if (warp < 4) {
            // ------------------------------ MMA issuers -----------------------------------
            // Issuer (a, e) = warp (2a + e) owns that accumulator: position (i, j) goes into it with the sign
            // At[a][i] * At[e][j]; At = [[1,1,1,0],[0,1,-1,-1]], so column e takes j = e..e+2 and row a takes
            // i = a..a+2: a = 0 is idle in phase C and a = 1 in phase A, where the issuer still follows the ring
            // (wait, arrive).  The whole warp walks the loop with warp-uniform values (warp index and tensor-memory
            // base were broadcast from lane 0), so that descriptors and addresses live in uniform registers; one
            // elected lane issues the MMAs and the commits.
            constexpr uint32_t idesc_pos = make_idesc_tf32(kBlockM, kBlockN);
            constexpr uint32_t idesc_neg = idesc_pos | (1u << 14);            // negate B
            const bool leader = elect_one();
            const int a = warp >> 1, e = warp & 1;
            const uint32_t d_tmem = tmem_base + (uint32_t)(warp * kBlockN);
            const uint32_t a_tmem0 = tmem_base + (uint32_t)kFuACol0;
            const uint64_t bdesc0 = make_desc_k_sw128(wbase), b2desc0 = make_desc_k_sw64(wbase);
            const uint32_t b_hi = (uint32_t)(bdesc0 >> 32), b_lo0 = (uint32_t)bdesc0;
            const uint32_t b2_hi = (uint32_t)(b2desc0 >> 32), b2_lo0 = (uint32_t)b2desc0;
            const int my_units = (prm.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
            const int total = my_units * spu_slots;
            const int first_slot = a == 0 ? 0 : nC32, last_slot = a == 0 ? 3 * nC32 - 1 : 4 * nC32 - 1;   // of this accumulator, in a unit
            int g = 0; uint32_t gph = 0;
            int sl = 0;                                                       // slot within the unit
            uint32_t units_done = 0;
            int trm = 0; (void)trm;
            // this issuer's copy of the unit's sixteen zero-block words (bit cc: the [64 x 32] weight tile of position t,
            // input channels cc*32.., holds a non-zero)
            unsigned long long *my_masks = reinterpret_cast<unsigned long long *>(bars_gen + 32 + warp * 16);
            const uint32_t *my_masks32 = reinterpret_cast<const uint32_t *>(my_masks);
            bool dense = true;
            for (int n = 0; n < total; ++n) {
                if (sl == 0) {
                    int gu, rbu, segu, kbu;
                    decode((int)blockIdx.x + (int)units_done * (int)gridDim.x, gu, rbu, segu, kbu);
                    unsigned long long all = ~0ull;
                    __syncwarp();
                    if (lane < 16) {
                        all = __ldg(prm.masks + (long long)lane * prm.nKB + kbu);
                        my_masks[lane] = all;
                    }
                    const unsigned long long need = nC32 >= 64 ? ~0ull : ((1ull << nC32) - 1ull);
                    dense = __all_sync(0xffffffffu, (all & need) == need);   // the common case: no block of this unit is empty
                }
                if (warp == 0 && leader) TC_TRACE(1024 + 5 * trm);
                if (!mbar_wait_warp(full_bar(g), gph, abort_flag, 0x1000u | (warp << 8) | g, prm.spin_limit)) break;
                if (warp == 0 && leader) TC_TRACE(1024 + 5 * trm + 1);
                // this accumulator's first MMA of the unit overwrites it: the epilogue must have read the previous unit's
                if (sl == first_slot && !mbar_wait_warp(acce_bar(a), (units_done & 1u) ^ 1u, abort_flag, 0x1400u | (warp << 8) | a, prm.spin_limit)) break;
                if (warp == 0 && leader) TC_TRACE(1024 + 5 * trm + 2);
                tc_fence_after();
                const int phase = sl < nC32 ? 0 : (sl < 3 * nC32 ? 1 : 2);
                const bool active = phase == 1 || phase == 2 * a;
                const uint32_t a_tmem = a_tmem0 + (uint32_t)(g * kFuGroupCols);
                if (active && phase != 1) {
                    // one Winograd row, 32 channels: tile j at columns j*32, its two 16-channel halves 16 columns apart
                    const int i = phase == 0 ? 0 : 3, cc = phase == 0 ? sl : sl - 3 * nC32;
                    const bool neg_a = phase == 2;                                    // At[1][3] = -1, At[0][0] = +1
                    const uint32_t b_lo = b_lo0 + (uint32_t)(g * (kFuWBytes >> 4));
#pragma unroll
                    for (int jj = 0; jj < 3; ++jj) {
                        // an all-zero weight tile adds nothing (the unit's first chunk always runs: it zero-initialises)
                        if (!dense && cc > 0 && cc < 64 && !((my_masks32[2 * (4 * i + e + jj) + (cc >> 5)] >> (cc & 31)) & 1u)) continue;
                        const bool neg_e = (e == 1 && jj >= 1);                      // At[1][j] = -1 for j = 2, 3
                        const uint32_t idesc = (neg_a != neg_e) ? idesc_neg : idesc_pos;
                        const uint32_t aj = a_tmem + (uint32_t)((e + jj) * 32), bj = b_lo + (uint32_t)((e + jj) * (kFuWTile >> 4));
#ifndef WG_KO_MMA  // (development knock-out: no MMAs, results wrong)
                        if (leader) {
                            umma_tf32_ts_x2(d_tmem, aj, bj, b_hi, idesc, (jj == 0 && sl == first_slot) ? 0u : 1u);
                            umma_tf32_ts_x2(d_tmem, aj + 16u, bj + 4u, b_hi, idesc, 1u);
                        }
#endif
                    }
                } else if (active) {
                    // Winograd rows 1 and 2, 16 channels: tile (i - 1) * 4 + j at columns 16 * tile, weights in rows of 64 bytes
                    const int c16 = sl - nC32, cc = c16 >> 1;
                    const uint32_t b_lo = b2_lo0 + (uint32_t)(g * (kFuWBytes >> 4));
#pragma unroll
                    for (int ii = 1; ii <= 2; ++ii) {
                        const bool neg_a = (a == 1 && ii == 2);                          // At[1][2] = -1
#pragma unroll
                        for (int jj = 0; jj < 3; ++jj) {
                            if (!dense && cc > 0 && cc < 64 && !((my_masks32[2 * (4 * ii + e + jj) + (cc >> 5)] >> (cc & 31)) & 1u)) continue;
                            const bool neg_e = (e == 1 && jj >= 1);
                            const uint32_t idesc = (neg_a != neg_e) ? idesc_neg : idesc_pos;
                            const int tile = (ii - 1) * 4 + e + jj;
                            const uint32_t aj = a_tmem + (uint32_t)(tile * 16), bj = b_lo + (uint32_t)(tile * (kFuW2Tile >> 4));
#ifndef WG_KO_MMA
                            if (leader) umma_tf32_ts_x2(d_tmem, aj, bj, b2_hi, idesc, (ii == 1 && jj == 0 && sl == first_slot) ? 0u : 1u);
#endif
                        }
                    }
                }
                if (warp == 0 && leader) TC_TRACE(1024 + 5 * trm + 3);
                if (leader) {
                    // (an issuer that added nothing in this slot has nothing for a commit to track: it arrives directly)
                    if (active) umma_commit(free_bar(g)); else mbar_arrive(free_bar(g));
                    if (sl == last_slot) umma_commit(accf_bar(a));                   // this accumulator is complete
                }
                __syncwarp();
                if (warp == 0 && leader) { TC_TRACE(1024 + 5 * trm + 4); ++trm; }
                if (++g == kFuAGroups) { g = 0; gph ^= 1u; }
                if (++sl == spu_slots) { sl = 0; ++units_done; }
            }
        } else if (warp == 4 && lane == 0) {
            // ------------------------------ X producer -----------------------------------
            int xb = 0, xj = 0; uint32_t xph = 0;               // buffer n % XB (xempty phase parity xph), barrier xfull[n % (2*XB)]
            bool ok = true;
            int trx = 0; (void)trx;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int g, rb, seg, kb;
                decode(u, g, rb, seg, kb);
                const int x0 = 2 * seg * prm.TW - 4, th0 = rb * prm.TH, b0 = g * prm.NB;
                for (int st = 0; st < 2 * spu_slots; ++st) {       // channels beyond C arrive as zeros
                    if (!mbar_wait_sleepy(xempty_bar(xb), xph ^ 1u, abort_flag, 0x900u | xb, 100, prm.spin_limit)) { ok = false; break; }
                    TC_TRACE(trx); ++trx;
                    const uint32_t dst = xbase + xb * kFuXbufBytes;
#ifdef WG_KO_X     // development knock-out: no input loads (results wrong)
                    mbar_arrive(xfull_bar(xj)); (void)dst; (void)x0; (void)th0; (void)b0;
#else
                    if (st >= 2 * nC32 && st < 6 * nC32) {         // phase B: rows d1, d2 of 8 channels, dense
                        mbar_expect_tx(xfull_bar(xj), prm.xbytes1);
                        tma_load_4d(dst, &mapXd, xfull_bar(xj), x0, 2 * th0, (st - 2 * nC32) * 8, b0);
                    } else {                                       // phase A: rows d0, d2; phase C: rows d1, d3 (every second row)
                        const bool first = st < 2 * nC32;
                        mbar_expect_tx(xfull_bar(xj), prm.xbytes2);
                        tma_load_4d(dst, &mapXs, xfull_bar(xj), x0, 2 * th0 - (first ? 1 : 0), (first ? st : st - 6 * nC32) * 16, b0);
                    }
#endif
                    if (++xb == kFuXbufs) { xb = 0; xph ^= 1u; }
                    if (++xj == kFuXfull) xj = 0;
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        } else if (warp == 6 && lane == 0) {
            // ------------------------------ W producer -----------------------------------
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            int nload = 0;
            for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
                int g, rb, seg, kb;
                decode(u, g, rb, seg, kb);
                for (int sl = 0; sl < spu_slots; ++sl) {
                    if (!mbar_wait_sleepy(free_bar(s), ph ^ 1u, abort_flag, 0xA00u | s, 100, prm.spin_limit)) { ok = false; break; }
                    // test hook: this slot's weights never arrive (nothing is put in flight), so the issuers' wait on it runs out
                    if (blockIdx.x == 0 && nload++ == prm.drop_load) { ok = false; break; }
#ifdef WG_KO_W     // development knock-out: no weight loads (results wrong)
                    mbar_arrive(full_bar(s));
#else
                    mbar_expect_tx(full_bar(s), kFuWBytes);
                    if (sl < nC32)          tma_load_3d(wbase + s * kFuWBytes, &mapW, full_bar(s), sl * 32, kb * kBlockN, 0);
                    else if (sl < 3 * nC32) tma_load_3d(wbase + s * kFuWBytes, &mapW2, full_bar(s), (sl - nC32) * 16, kb * kBlockN, 4);
                    else                    tma_load_3d(wbase + s * kFuWBytes, &mapW, full_bar(s), (sl - 3 * nC32) * 32, kb * kBlockN, 12);
#endif
                    if (++s == kFuWStages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        }
    } else if (warp >= 16) {
        // ------------------------------ transform teams ----------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kFuRegsXf));
        const int team = (warp - 16) / kFuTeamWarps;
        const int tw8 = (warp - 16) % kFuTeamWarps;
        const int l = (tw8 & 3) * 32 + lane;                   // tile = TMEM lane = A-tile row
        const int hq = tw8 >> 2;                               // which half of the step's channels
        // a tile row occupies LP = 2^lp_log2 >= TW consecutive lanes, so it never straddles a warp (or, for
        // LP <= 16, a half-warp: the 8-byte loads of a half-warp then stay conflict-free)
        const int trow = l >> prm.lp_log2, tcol = l & ((1 << prm.lp_log2) - 1);
        const bool live = tcol < prm.TW && trow < prm.NB * prm.TH;
        // The outer two pixels of a tile's window are the neighbouring tiles' middle ones and come by a rotation
        // among the lanes of the tile row.  Dead lanes (their A rows feed TMEM lanes nobody reads) work for their
        // neighbours: with at least two of them per tile row, the first reads the pixel pair right of the last tile
        // and the last one the pair left of the first tile; otherwise the lanes at the ends load their outer pixel.
        // Rows beyond the block shadow row 0.
        const int LP = 1 << prm.lp_log2;
        const bool halo_by_lanes = LP - prm.TW >= 2;
        const int row_e = trow < prm.NB * prm.TH ? trow : 0;
        const int twl = halo_by_lanes ? ((tcol == LP - 1) ? -1 : (tcol < prm.TW ? tcol : prm.TW)) : (live ? tcol : 0);
        const int bi = row_e / prm.TH, thl = row_e - bi * prm.TH;
        const int BW = prm.BW;
        const int src_l = (lane & ~(LP - 1)) | ((tcol + LP - 1) & (LP - 1)), src_r = (lane & ~(LP - 1)) | ((tcol + 1) & (LP - 1));
        const bool need_l = !halo_by_lanes && (tcol == 0), need_r = !halo_by_lanes && ((tcol == prm.TW - 1) || (tcol == LP - 1));
        const float lo = prm.relu ? 0.f : -__int_as_float(0x7f800000);
        const int spu = 2 * spu_slots;                          // steps per unit
        const int my_units = (prm.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const int total = my_units * spu;
        // Steps 2s and 2s+1 fill the two halves of ring slot s (A group s % 2).  This team takes the steps
        // n = 2k + team, i.e. its own half of every slot, so the two teams work on a slot side by side and both
        // see every phase of the slot's barriers.  X buffer n % kFuXbufs, full-barrier n % kFuXfull.
        static_assert(kFuAGroups == 2 && kFuXfull % 2 == 0, "each xfull barrier belongs to one team");
        bool ok = true;
        int trt = 0; (void)trt;
        // running values of n % kFuXfull (and its wrap parity) and of the step within the unit
        int xj = team, st = team;
        uint32_t xph = 0;
        // AFFINE: the image is s_c * x + t_c inside and 0 in the padding, so B^T d B = s_c * (B^T x B) + t_c * R_i * C_j
        // with R = B^T rowmask, C = B^T colmask of the tile's 4 x 4 window (R = C = (0,2,0,0) away from the border)
        int unit = blockIdx.x;
        float Rm[4] = {0.f, 0.f, 0.f, 0.f}, Cm[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0, n = team; n < total; ++k, n += 2) {
            if (AFFINE && st == team) {
                int gu, rbu, segu, kbu;
                decode(unit, gu, rbu, segu, kbu);
                unit += gridDim.x;
                const int y0 = 2 * (rbu * prm.TH + thl) - 1, x0w = 2 * (segu * prm.TW + tcol) - 1;
                float mr[4], mc[4];
#pragma unroll
                for (int d = 0; d < 4; ++d) {
                    mr[d] = (y0 + d >= 0 && y0 + d < prm.H) ? 1.f : 0.f;
                    mc[d] = (x0w + d >= 0 && x0w + d < prm.W) ? 1.f : 0.f;
                }
                Rm[0] = mr[0] - mr[2]; Rm[1] = mr[1] + mr[2]; Rm[2] = mr[2] - mr[1]; Rm[3] = mr[1] - mr[3];
                Cm[0] = mc[0] - mc[2]; Cm[1] = mc[1] + mc[2]; Cm[2] = mc[2] - mc[1]; Cm[3] = mc[1] - mc[3];
            }
            const int g = k & 1;
            const uint32_t gph = (uint32_t)(k >> 1) & 1u;          // slot k is this group's (k / 2)-th filling
            const int xb = xj < kFuXbufs ? xj : xj - kFuXbufs;
            const int phase = st < 2 * nC32 ? 0 : (st < 6 * nC32 ? 1 : 2);
            const bool mid = phase == 1;                         // rows 1 and 2 together, from input rows d1 and d2
            // first channel of the step and the thread's first channel within it (8 per thread, 4 in phase B)
            const int ch_step = mid ? (st - 2 * nC32) * 8 : (phase == 0 ? st : st - 6 * nC32) * 16;
            const int ch_mine = mid ? 4 * hq : 8 * hq;
            const int rows = mid ? 2 * prm.TH : prm.TH + 1;      // rows of a channel in the X buffer
            const int nch = mid ? 8 : 16;                        // channels of an image in the X buffer
            const int ra = mid ? 2 * thl : thl;                  // first of the tile's two input rows; the second is the next one
            const float sb = phase == 0 ? -1.f : (phase == 2 ? -1.f : 1.f);   // phase A: d0 - d2; phase C: d1 - d3
            // AFFINE: the shift term of a value is t_c * R_i * C_j
            float RCa[4], RCb[4];                                // row i = 0 / 3 (or 1 in phase B), and row 2 in phase B
            if (AFFINE) {
                const float Ri = phase == 0 ? Rm[0] : (phase == 2 ? Rm[3] : Rm[1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) { RCa[j] = Ri * Cm[j]; RCb[j] = Rm[2] * Cm[j]; }
            }
            // AFFINE: this thread's channels' scale and shift, fetched before the waits so that their latency hides there
            float sc8[8], tc8[8];
            if (AFFINE) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int chg = ch_step + ch_mine + c;
                    const bool in = chg < prm.C && (c < 4 || !mid);
                    sc8[c] = in ? __ldg(prm.in_scale + chg) : 0.f;
                    tc8[c] = in ? __ldg(prm.in_shift + chg) : 0.f;
                }
            }
            if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt);
            // both waits, then one vote (the warp converged and of one mind before the aligned instructions below)
            const bool got_x = mbar_wait(xfull_bar(xj), xph, abort_flag, 0xB00u | xj, prm.spin_limit);
            if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 1);
            const bool got_a = got_x && mbar_wait(free_bar(g), gph ^ 1u, abort_flag, 0xC00u | g, prm.spin_limit);
            if (!__all_sync(0xffffffffu, got_a)) { ok = false; break; }
            if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 2);
            const int chs = rows * BW;
            const int off0 = ((bi * nch + ch_mine) * rows + ra) * BW + 2 * twl;
            const float *xq = xgen + xb * (kFuXbufBytes / 4) + off0 + 3;
            const uint32_t xq_s = xbase + (uint32_t)(xb * kFuXbufBytes + 4 * (off0 + 4));   // the 8-byte loads, shared-space address
            tc_fence_after();
            const uint32_t a_grp = tmem_base + ((uint32_t)((tw8 & 3) * 32) << 16) + (uint32_t)(kFuACol0 + g * kFuGroupCols);
            // the row combination a + sb * b of the tile's four window pixels: the middle two from one 8-byte load per
            // input row, the outer two from the neighbouring lanes
            auto window = [&](auto by_lanes_tag, int c, float s2, float &r0, float &r1, float &r2, float &r3) {
                constexpr bool kByLanes = decltype(by_lanes_tag)::value;
                const float *pa = xq + c * chs;
                const float *pb = pa + BW;
#ifdef WG_KO_LDS   // development knock-out: no shared-memory loads (results wrong)
                const float2 am = make_float2((float)c, s2), bm = make_float2(s2, 1.f);
#else
                const float2 am = lds_f2(xq_s + (uint32_t)(4 * c * chs));
                const float2 bm = lds_f2(xq_s + (uint32_t)(4 * (c * chs + BW)));
#endif
                r1 = fmaf(s2, bm.x, am.x); r2 = fmaf(s2, bm.y, am.y);
#ifdef WG_KO_SHFL  // development knock-out: no shuffles (results wrong)
                r0 = r2 * 0.5f; r3 = r1 * 0.25f;
#else
                r0 = __shfl_sync(0xffffffffu, r2, src_l); r3 = __shfl_sync(0xffffffffu, r1, src_r);
#endif
                if (!kByLanes) {
                    if (need_l) r0 = fmaf(s2, pb[0], pa[0]);
                    if (need_r) r3 = fmaf(s2, pb[3], pa[3]);
                }
            };
            auto body = [&](auto by_lanes_tag) {
                if (!mid) {
                    // one Winograd row of 16 channels: this thread's 8 channels as two quads, tile j at columns j*32
                    const uint32_t a_tmem = a_grp + (uint32_t)(team * 16);
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int c4 = 2 * hq + q;
                        float o[4][4];   // [j][channel within the quad]
#pragma unroll
                        for (int cq = 0; cq < 4; ++cq) {
                            float r0, r1, r2, r3;
                            window(by_lanes_tag, q * 4 + cq, sb, r0, r1, r2, r3);
                            // (fp32 values; what the tensor core makes of the low mantissa bits: see tmem_st4)
                            if (AFFINE) {
                                const float sc = sc8[q * 4 + cq], tc = tc8[q * 4 + cq];
                                o[0][cq] = fmaxf(fmaf(sc, r0 - r2, tc * RCa[0]), lo);
                                o[1][cq] = fmaxf(fmaf(sc, r1 + r2, tc * RCa[1]), lo);
                                o[2][cq] = fmaxf(fmaf(sc, r2 - r1, tc * RCa[2]), lo);
                                o[3][cq] = fmaxf(fmaf(sc, r1 - r3, tc * RCa[3]), lo);
                            } else {
                                o[0][cq] = fmaxf(r0 - r2, lo);
                                o[1][cq] = fmaxf(r1 + r2, lo);
                                o[2][cq] = fmaxf(r2 - r1, lo);
                                o[3][cq] = fmaxf(r1 - r3, lo);
                            }
                        }
#ifdef WG_KO_ST    // development knock-out: one tensor-memory store instead of four (results wrong)
                        { float z[4] = {o[0][0] + o[1][1], o[2][2] + o[3][3], o[0][1] + o[1][2], o[2][3] + o[3][0]}; tmem_st4(a_tmem + (uint32_t)(c4 * 4), z); }
#else
#pragma unroll
                        for (int j = 0; j < 4; ++j) tmem_st4(a_tmem + (uint32_t)(j * 32 + c4 * 4), o[j]);
#endif
                        if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 4 + q);
                    }
                } else {
                    // Winograd rows 1 and 2 of 8 channels: this thread's 4 channels, tile (i - 1) * 4 + j at columns 16 * tile
                    const uint32_t a_tmem = a_grp + (uint32_t)(team * 8 + hq * 4);
                    // the middle pixels of both rows from one pair of loads per channel
                    float m1[4][2], m2[4][2], e1[4][2], e2[4][2];   // [channel][left, right]: rows 1 and 2; e*: the outer pixels where lanes cannot supply them
#pragma unroll
                    for (int cq = 0; cq < 4; ++cq) {
#ifdef WG_KO_LDS   // development knock-out: no shared-memory loads (results wrong)
                        const float2 am = make_float2((float)cq, lo), bm = make_float2(lo, 1.f);
#else
                        const float2 am = lds_f2(xq_s + (uint32_t)(4 * cq * chs));
                        const float2 bm = lds_f2(xq_s + (uint32_t)(4 * (cq * chs + BW)));
#endif
                        m1[cq][0] = am.x + bm.x; m1[cq][1] = am.y + bm.y;      // row 1 = d1 + d2
                        m2[cq][0] = bm.x - am.x; m2[cq][1] = bm.y - am.y;      // row 2 = d2 - d1
                        if (!decltype(by_lanes_tag)::value) {
                            const float *pa = xq + cq * chs, *pb = pa + BW;
                            e1[cq][0] = pa[0] + pb[0]; e1[cq][1] = pa[3] + pb[3];
                            e2[cq][0] = pb[0] - pa[0]; e2[cq][1] = pb[3] - pa[3];
                        }
                    }
#pragma unroll
                    for (int ii = 0; ii < 2; ++ii) {
                        float o[4][4];   // [j][channel]
#pragma unroll
                        for (int cq = 0; cq < 4; ++cq) {
                            const float r1 = ii == 0 ? m1[cq][0] : m2[cq][0], r2 = ii == 0 ? m1[cq][1] : m2[cq][1];
#ifdef WG_KO_SHFL  // development knock-out: no shuffles (results wrong)
                            float r0 = r2 * 0.5f, r3 = r1 * 0.25f;
#else
                            float r0 = __shfl_sync(0xffffffffu, r2, src_l), r3 = __shfl_sync(0xffffffffu, r1, src_r);
#endif
                            if (!decltype(by_lanes_tag)::value) {
                                if (need_l) r0 = ii == 0 ? e1[cq][0] : e2[cq][0];
                                if (need_r) r3 = ii == 0 ? e1[cq][1] : e2[cq][1];
                            }
                            if (AFFINE) {
                                const float sc = sc8[cq], tc = tc8[cq];
                                o[0][cq] = fmaxf(fmaf(sc, r0 - r2, tc * (ii == 0 ? RCa[0] : RCb[0])), lo);
                                o[1][cq] = fmaxf(fmaf(sc, r1 + r2, tc * (ii == 0 ? RCa[1] : RCb[1])), lo);
                                o[2][cq] = fmaxf(fmaf(sc, r2 - r1, tc * (ii == 0 ? RCa[2] : RCb[2])), lo);
                                o[3][cq] = fmaxf(fmaf(sc, r1 - r3, tc * (ii == 0 ? RCa[3] : RCb[3])), lo);
                            } else {
                                o[0][cq] = fmaxf(r0 - r2, lo);
                                o[1][cq] = fmaxf(r1 + r2, lo);
                                o[2][cq] = fmaxf(r2 - r1, lo);
                                o[3][cq] = fmaxf(r1 - r3, lo);
                            }
                        }
#ifdef WG_KO_ST    // development knock-out: one tensor-memory store instead of four (results wrong)
                        { float z[4] = {o[0][0] + o[1][1], o[2][2] + o[3][3], o[0][1] + o[1][2], o[2][3] + o[3][0]}; tmem_st4(a_tmem + (uint32_t)(ii * 64), z); }
#else
#pragma unroll
                        for (int j = 0; j < 4; ++j) tmem_st4(a_tmem + (uint32_t)((4 * ii + j) * 16), o[j]);
#endif
                        if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 4 + ii);
                    }
                }
            };
            // (two copies, so that the common case carries no test for the lanes at the ends of a tile row)
            if (halo_by_lanes) body(std::true_type{}); else body(std::false_type{});
            // the tensor-memory writes have to be complete before the MMA issuers are told
            tmem_st_wait();
            if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 6);
            tc_fence_before();
            __syncwarp();
            if (warp == 16 && lane == 0) TC_TRACE(512 + 8 * trt + 3);
            ++trt;
            if (lane == 0) {
                mbar_arrive(full_bar(g));
                mbar_arrive(xempty_bar(xb));
            }
            xj += 2; if (xj >= kFuXfull) { xj -= kFuXfull; xph ^= 1u; }
            st += 2; if (st >= spu) st -= spu;
        }
        (void)ok;
    } else {
        // ------------------------------ epilogue ------------------------------------------
        const int ew = warp - 8;                                 // (these warps keep the 64 registers of the launch)
        const int q = warp & 3;
        const int half = ew >> 2;                                // which 32 of the 64 output channels
        const int l = q * 32 + lane;
        const int trow = l >> prm.lp_log2, tcol = l & ((1 << prm.lp_log2) - 1);   // same lane <-> tile map as the transform warps
        const bool live = tcol < prm.TW && trow < prm.NB * prm.TH;
        const int row_e = live ? trow : 0, twl = live ? tcol : 0;
        const int bi = row_e / prm.TH, thl = row_e - bi * prm.TH;
        const int BWY = prm.BWY, TH = prm.TH;
        float *stage0 = reinterpret_cast<float *>(gen_base + kYOff + half * kFuYBoxes * kFuYStageBytes);
        const int my_off = (bi * 16 * TH + thl) * BWY + 2 * twl; // this thread's tile in channel 0 of a box
        const bool elected = ((ew & 3) == 0) && lane == 0;
        uint32_t units_done = 0, st_use = 0;
        int ybox = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < prm.units && ok; u += gridDim.x) {
            int g, rb, seg, kb;
            decode(u, g, rb, seg, kb);
            const int kbase = kb * kBlockN + half * 32;
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                if (ew == 0 && lane == 0) TC_TRACE(2048 + 4 * (int)units_done + 2 * a);
                if (!__all_sync(0xffffffffu, mbar_wait_sleepy(accf_bar(a), units_done & 1u, abort_flag, 0x400u | (ew << 4) | a, 400, prm.spin_limit))) { ok = false; break; }
                if (ew == 0 && lane == 0) TC_TRACE(2048 + 4 * (int)units_done + 2 * a + 1);
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * 2 * kBlockN + half * 32);
#pragma unroll
                for (int rd = 0; rd < 2; ++rd) {
                    float v0[16], v1[16];                         // pixels (a, 0) and (a, 1) of 16 channels
                    tmem_ld8(taddr + (uint32_t)(rd * 16), v0);
                    tmem_ld8(taddr + (uint32_t)(rd * 16 + 8), v0 + 8);
                    tmem_ld8(taddr + (uint32_t)(kBlockN + rd * 16), v1);
                    tmem_ld8(taddr + (uint32_t)(kBlockN + rd * 16 + 8), v1 + 8);
                    tmem_ld_wait();
                    if (rd == 1) {                                // output row a is in registers: hand its accumulators back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acce_bar(a));
                    }
                    // the store that last used this staging box has left it (all but the kFuYBoxes - 1 most recent stores have been read)
                    if (elected) {
                        asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kFuYBoxes - 1) : "memory");
                        mbar_arrive(yfree_bar(half));
                    }
                    if (!mbar_wait_warp(yfree_bar(half), st_use & 1u, abort_flag, 0x500u | ew, prm.spin_limit)) { ok = false; break; }
                    float *stage = stage0 + ybox * (kFuYStageBytes / 4);
#ifdef WG_KO_Y     // development knock-out: Y is neither staged nor stored (results wrong)
                    if (false) {
#else
                    if (live) {
#endif
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int k = kbase + rd * 16 + c;
                            float y0 = v0[c], y1 = v1[c];
                            if (EXTRAS && k < prm.K) {
                                if (prm.out_scale) {
                                    const float s1 = __ldg(prm.out_scale + k), b1 = __ldg(prm.out_shift + k);
                                    y0 = fmaf(y0, s1, b1); y1 = fmaf(y1, s1, b1);
                                }
                            }
                            *reinterpret_cast<float2 *>(stage + my_off + c * TH * BWY) = make_float2(y0, y1);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ywritten_bar(half));
                    bool stored = true;
                    if (elected) {
                        stored = mbar_wait(ywritten_bar(half), st_use & 1u, abort_flag, 0x580u | ew, prm.spin_limit);
#ifdef WG_KO_Y
                        if (false) {
#else
                        if (stored && kbase + rd * 16 < prm.K) {      // a box that starts beyond the last channel is not issued at all
#endif
                            if (prm.accumulate) tma_reduce_add_4d(smem_u32(stage), &mapY, 2 * seg * prm.TW, 2 * rb * TH + a, kbase + rd * 16, g * prm.NB);
                            else tma_store_4d(smem_u32(stage), &mapY, 2 * seg * prm.TW, 2 * rb * TH + a, kbase + rd * 16, g * prm.NB);
                        }
                        // (an empty group when nothing was issued: the count of groups per round stays the same)
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    // the warp goes on together (tcgen05.ld is next) and with one outcome
                    if (!__all_sync(0xffffffffu, stored)) { ok = false; break; }
                    ++st_use;
                    if (++ybox == kFuYBoxes) ybox = 0;
                }
                if (!ok) break;
            }
            ++units_done;
        }
        // the last boxes must have reached memory before the CTA ends
        if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    __syncwarp();                        // the lanes of a warp took different roles: together again before the aligned instructions
    tc_fence_before();
    __syncthreads();
    FU_CTA_STAMP(2);
    if (warp == 1) {
        __syncwarp();
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
    p.BWY = (2 * p.TW + 3) & ~3;
    // the larger of the two input boxes ((TH + 1) rows x BW x 16 channels x NB images; the dense one has 2*TH rows of 8
    // channels) has to fit an X buffer, and the output box (TH rows x BWY x 16 channels x NB images) a staging box
    auto fits = [&](int th, int nb) {
        return (size_t)p.BW * (th + 1) * 16 * 4 * nb <= (size_t)kFuXbufBytes && (size_t)p.BWY * th * 16 * 4 * nb <= (size_t)kFuYStageBytes;
    };
    p.lp_log2 = 0;
    while ((1 << p.lp_log2) < p.TW) ++p.lp_log2;
    const int max_rows = kBlockM >> p.lp_log2;              // tile rows (of all images) per unit
    int TH = max_rows;
    if (TH > p.nH) TH = p.nH;
    while (TH > 1 && !fits(TH, 1)) --TH;
    if (!fits(TH, 1)) return false;
    p.nRB = cdiv(p.nH, TH);
    TH = cdiv(p.nH, p.nRB);                  // same number of row blocks, evened out
    p.TH = TH;
    p.NB = 1;
    if (TH == p.nH) {
        int nb = max_rows / TH;
        while (nb > 1 && !fits(TH, nb)) --nb;
        if (nb > p.B) nb = p.B;
        p.NB = nb < 1 ? 1 : nb;
    }
    if (2 * (TH + 1) > 256) return false;    // TMA box extent
    p.nGroups = cdiv(p.B, p.NB);
    p.nKB = cdiv(p.K, kBlockN);
    p.nC32 = cdiv(p.C, 32);
    p.xbytes1 = (uint32_t)((size_t)p.BW * 2 * TH * 8 * p.NB * 4);
    p.xbytes2 = (uint32_t)((size_t)p.BW * (TH + 1) * 16 * p.NB * 4);
    const long long units = (long long)p.nGroups * p.nRB * p.nSeg * p.nKB;
    if (units > 0x7fffffffLL) return false;
    p.units = (int)units;
    return true;
}

int layer_fwd_fused(const float *X, const void *prepared, float *Y, int B, int H, int W, int C, int K, int relu,
                    const float *in_scale, const float *in_shift, const float *out_scale, const float *out_shift,
                    const float *residual, cudaStream_t st)
{
    if (!X || !prepared || !Y) return WG2X2_ERR_BAD_ARG;
    if ((in_scale == nullptr) != (in_shift == nullptr)) return WG2X2_ERR_BAD_ARG;
    if (!fused_fwd_supported(B, H, W, C, K, WG2X2_NCHW)) return WG2X2_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (reinterpret_cast<uintptr_t>(Y) & 15u)) return WG2X2_ERR_BAD_ARG;
    if ((out_scale == nullptr) != (out_shift == nullptr)) return WG2X2_ERR_BAD_ARG;
    FuParams p;
    p.Y = Y; p.out_scale = out_scale; p.out_shift = out_shift;
    // The shortcut is added by the TMA unit: Y receives it first (unless it is Y already), then every box is reduced
    // into Y instead of stored.
    p.accumulate = residual != nullptr;
    if (residual && residual != Y &&
        cudaMemcpyAsync(Y, residual, sizeof(float) * (size_t)B * K * H * W, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return WG2X2_ERR_LAUNCH;
    p.in_scale = in_scale; p.in_shift = in_shift;
    p.masks = reinterpret_cast<const unsigned long long *>(static_cast<const unsigned char *>(prepared) +
                                                           align_up((size_t)16 * K * C * sizeof(float), 256));
    p.B = B; p.H = H; p.W = W; p.C = C; p.K = K; p.outH = H; p.outW = W; p.relu = relu;
    if (!fused_geometry(p)) return WG2X2_ERR_UNSUPPORTED;
    p.spin_limit = wait_limit();
    p.drop_load = take_drop_load();
    EncodeTiledFn fn = encode_fn();
    if (!fn) return WG2X2_ERR_LAUNCH;
    CUtensorMap mapX1, mapX2, mapW, mapW2, mapY;
    {
        cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)B};
        cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4, (cuuint64_t)C * H * W * 4};
        // dense box of 8 channels: rows 2*th0 .. 2*th0 + 2*TH - 1
        cuuint32_t box1[4] = {(cuuint32_t)p.BW, (cuuint32_t)(2 * p.TH), 8, (cuuint32_t)p.NB};
        cuuint32_t estr1[4] = {1, 1, 1, 1};
        if (fn(&mapX1, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(X), dims, strides, box1, estr1,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
        // every second row: a box extent of 2*(TH+1) walked with stride 2 brings TH+1 rows
        cuuint32_t box2[4] = {(cuuint32_t)p.BW, (cuuint32_t)(2 * (p.TH + 1)), 16, (cuuint32_t)p.NB};
        cuuint32_t estr2[4] = {1, 2, 1, 1};
        if (fn(&mapX2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(X), dims, strides, box2, estr2,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)K, 16};
        cuuint64_t strides[2] = {(cuuint64_t)C * 4, (cuuint64_t)K * C * 4};
        cuuint32_t box[3] = {32, (cuuint32_t)kBlockN, 4};
        cuuint32_t estr[3] = {1, 1, 1};
        if (fn(&mapW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(prepared), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
        // phase B: the eight positions of Winograd rows 1 and 2, 16 channels each, rows of 64 bytes (64-byte swizzle)
        cuuint32_t box2[3] = {16, (cuuint32_t)kBlockN, 8};
        if (fn(&mapW2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(prepared), dims, strides, box2, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)K, (cuuint64_t)B};
        cuuint64_t strides[3] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4, (cuuint64_t)K * H * W * 4};
        // output rows of one parity: a box extent of 2*TH walked with stride 2 is TH rows
        cuuint32_t box[4] = {(cuuint32_t)p.BWY, (cuuint32_t)(2 * p.TH), 16, (cuuint32_t)p.NB};
        cuuint32_t estr[4] = {1, 2, 1, 1};
        if (fn(&mapY, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Y, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return WG2X2_ERR_LAUNCH;
    }
    // a grid that divides the units evenly: every CTA runs the same number of them
    const int rounds = cdiv(p.units, kNumSMs);
    const int grid = cdiv(p.units, rounds);
    const bool extras = out_scale != nullptr, affine = in_scale != nullptr;
    // Back-to-back layers: the next launch's scheduling and set-up overlap this kernel's tail (programmatic dependent
    // launch; the kernel waits for its predecessor before its first global access).  Not while a graph is being
    // captured, and WG2X2_PDL=0 in the environment turns it off.
    static const bool pdl_env = [] { const char *e = getenv("WG2X2_PDL"); return !(e && e[0] == '0'); }();
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess) return WG2X2_ERR_LAUNCH;
    const bool pdl = pdl_env && capturing == cudaStreamCaptureStatusNone;
    auto launch = [&](auto kernel) -> bool {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFuSmemBytes) != cudaSuccess) return false;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3((unsigned)kFuThreads);
        cfg.dynamicSmemBytes = kFuSmemBytes; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
        return cudaLaunchKernelEx(&cfg, kernel, mapX1, mapX2, mapW, mapW2, mapY, p) == cudaSuccess;
    };
    const bool launched = extras ? (affine ? launch(layer_fwd_fused_kernel<true, true>) : launch(layer_fwd_fused_kernel<true, false>))
                                 : (affine ? launch(layer_fwd_fused_kernel<false, true>) : launch(layer_fwd_fused_kernel<false, false>));
    if (!launched) return WG2X2_ERR_LAUNCH;
    return launch_status();
}
