// The gradient / wide-forward GEMM on pairs of SMs (tcgen05 cta_group::2): two CTAs of a cluster share one 256 x N tile.
// Each CTA loads its own 128 rows of A and only HALF of the B tile (N/2 columns); the tensor cores of the two SMs
// exchange the halves, so that a CTA's shared memory sees 32 KB instead of 48 KB per 32 contraction steps, written once
// by TMA and read once by the MMAs: the traffic that bounds the one-CTA kernel (conv_grad_gemm_tc_kernel) at about
// 55 % of the tensor rate.  Included by conv_tc.cu after conv_tc_bwd.cuh, whose parameters, maps and epilogue it shares.
//
// Protocol (rank 0 of the pair = leader):
//   * both CTAs allocate their 512 tensor-memory columns with the cta_group::2 form (same warp, same slot address) and free
//     them after a cluster-wide barrier at the end;
//   * full[s] lives in the leader: its producer arms it with the bytes of BOTH CTAs' tiles, and the partner's TMA loads
//     complete on it as well (cta_group::2 loads, one destination each);
//   * the leader's MMA warp issues tcgen05.mma.cta_group::2 (M = 256) and commits twice, once to the barrier of each
//     CTA: empty[s] releases both producers, accf[b] wakes both epilogues;
//   * acce[b] lives in the leader and counts the epilogue warps of both CTAs (the partner's arrive remotely);
//   * every wait is bounded as elsewhere; a CTA that gives up still walks to the final cluster barrier.
#pragma once

constexpr int kGg2Stages = 6;
constexpr int kGg2StageBytes = kGgABytes + kGgBBytesMax / 2;   // 32 KB: 128 rows of A, 128 columns of B
constexpr int kGg2SmemBytes = kGg2Stages * kGg2StageBytes + 1024 + kCtrlBytes + kEpiWarps * kEpiStageBytes;
static_assert(kGg2SmemBytes <= 232448, "shared memory per CTA");

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// every thread of both CTAs
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the shared::cluster address of the same shared-memory location in the pair's leader
__device__ __forceinline__ uint32_t mapa_rank0(uint32_t addr)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(0u));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one CTA of a pair; the completion bytes go to a barrier that may sit in the partner
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// D[tmem of both CTAs] (+)= A * B, M = 256 (128 rows per CTA), K = 8 (tf32); issued by the leader only
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the shared::cluster address of the same shared-memory location in CTA `r` of the pair
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t r)
{
    uint32_t o;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(o) : "r"(addr), "r"(r));
    return o;
}
// the barrier at this offset in BOTH CTAs gets one arrival once all MMAs issued so far have completed (one commit each)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mapa_rank(bar, 0)) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mapa_rank(bar, 1)) : "memory");
}

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads, 1)
conv_grad_gemm_tc2_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                         const __grid_constant__ CUtensorMap mapOut, const GgParams prm)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (base - raw);
    const uint32_t bars = base + kGg2Stages * kGg2StageBytes;
    uint64_t *bars_gen = reinterpret_cast<uint64_t *>(gen_base + kGg2Stages * kGg2StageBytes);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kGg2Stages + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * kGg2Stages + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * kGg2Stages + 2 + b); };
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bars_gen + 2 * kGg2Stages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars_gen + 2 * kGg2Stages + 5);
    float *epi_stage_all = reinterpret_cast<float *>(gen_base + kGg2Stages * kGg2StageBytes + kCtrlBytes);

    // (broadcast from lane 0: the compiler then treats the warp index, and all that is derived from it, as warp-uniform)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();        // 0: the CTA that issues the pair's MMAs and owns the full / acce barriers
    if (threadIdx.x == 0) {
        // full: one arrival (the leader's expect_tx), bytes of both CTAs' loads; empty / accf: one arrival per CTA (the
        // leader's commit); acce (leader's only): the epilogue warps of both CTAs
        for (int s = 0; s < kGg2Stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 2 * kEpiWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {       // the same warp of both CTAs, the same slot address
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_ptr_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // the partner's barriers exist before anything is signalled into them
    tc_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_ptr_slot, 0);

    const int N = prm.N, NH = prm.N >> 1;          // each CTA holds half of the B tile's columns
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    // unit -> (split, t, pair of row blocks, column block); column block fastest so that neighbouring pairs share the A tiles in L2
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
            const uint32_t stage_tx = 2u * (uint32_t)(kGgABytes + NH * 128);   // both CTAs' tiles land on the leader's barrier
            for (int u = pair; u < prm.units && ok; u += npairs) {
                int split, t, rb, cb;
                decode(u, split, t, rb, cb);
                const long long kbeg = (long long)split * prm.chunks_per_split * 32;
                const long long kend = min(prm.contr, kbeg + (long long)prm.chunks_per_split * 32);
                const unsigned long long live = KIND == 1 ? gg_live_chunks(prm, t, cb) : ~0ull;
                for (long long kc = kbeg; kc < kend; kc += 32) {
                    if (KIND == 1 && kc < 64 * 32 && !((live >> (kc >> 5)) & 1ull)) continue;   // all-zero weight blocks: nothing to add
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 0x500u | s)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full_bar(s), stage_tx);
                    const uint32_t fbar = mapa_rank0(full_bar(s));
                    const uint32_t a_dst = base + s * kGg2StageBytes;
                    const uint32_t b_dst = a_dst + kGgABytes;
                    const int row0 = (2 * rb + (int)rank) * 128, col0 = cb * N + (int)rank * NH;
                    if (KIND == 0 && prm.mn4) {      // all 32-channel blocks of an operand in one box each
                        tma_load_4d_pair(a_dst, &mapA, fbar, 0, (int)kc, row0 / 32, t);
                        tma_load_4d_pair(b_dst, &mapB, fbar, 0, (int)kc, col0 / 32, t);
                    } else if (KIND == 0) {
#pragma unroll
                        for (int mb = 0; mb < 4; ++mb)
                            tma_load_3d_pair(a_dst + mb * kGgBoxBytes, &mapA, fbar, row0 + mb * 32, (int)kc, t);
                        for (int nb = 0; nb < NH / 32; ++nb)
                            tma_load_3d_pair(b_dst + nb * kGgBoxBytes, &mapB, fbar, col0 + nb * 32, (int)kc, t);
                    } else {
                        tma_load_3d_pair(a_dst, &mapA, fbar, (int)kc, row0, t);
                        tma_load_3d_pair(b_dst, &mapB, fbar, (int)kc, col0, t);
                    }
                    if (++s == kGg2Stages) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok)
                for (int it = 0; it < 1000; ++it) __nanosleep(1000);
        }
    } else if (warp == 1 && rank != 0) {
        // the partner's MMA warp only takes part in the allocation of tensor memory
    } else if (warp == 1) {
        // The whole warp walks the loop with warp-uniform values (descriptors and addresses in uniform registers); one
        // elected lane issues the MMAs and the commits.  Issued by a lone lane from per-thread registers, an MMA costs
        // several times as many issue slots, for which the eight epilogue warps compete.
        {
            const bool leader = elect_one();
            const uint32_t idesc = make_idesc_tf32(256, N) | (KIND == 0 ? ((1u << 15) | (1u << 16)) : 0u);
            int s = 0; uint32_t ph = 0;
            uint32_t acc_use[2] = {0, 0};
            int buf = 0;
            bool ok = true;
            for (int u = pair; u < prm.units && ok; u += npairs) {
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
                    const uint32_t a_addr = base + s * kGg2StageBytes;
                    const uint64_t adesc = KIND == 0 ? make_desc_mn_sw128(a_addr) : make_desc_k_sw128(a_addr);
                    const uint64_t bdesc = KIND == 0 ? make_desc_mn_sw128(a_addr + kGgABytes) : make_desc_k_sw128(a_addr + kGgABytes);
                    const uint32_t step = KIND == 0 ? 64u : 2u;   // 1024 B / 32 B per 8 contraction steps
                    if (leader) {
#pragma unroll
                        for (int kg = 0; kg < 4; ++kg)
                            umma_tf32_pair(d_tmem, adesc + step * kg, bdesc + step * kg, idesc, (first && kg == 0) ? 0u : 1u);
                        umma_commit_pair(empty_bar(s));
                    }
                    __syncwarp();
                    first = 0;
                    if (++s == kGg2Stages) { s = 0; ph ^= 1u; }
                }
                if (ok && leader) umma_commit_pair(accf_bar(buf));
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
        for (int u = pair; u < prm.units && ok; u += npairs) {
            int split, t, rb, cb;
            decode(u, split, t, rb, cb);
            const bool use_mask = prm.mask && (KIND == 1 || prm.direct);
            const int rb1 = 2 * rb + (int)rank;          // this CTA's 128 rows of the pair's 256
            const long long row = (long long)rb1 * 128 + q * 32 + lane;
            const long long row_off = (prm.direct ? 0 : (long long)split * plane_elems) + ((long long)t * prm.rows + row) * prm.cols;
            const int ncol_half = N / 2;
            for (int cc = 0; cc < ncol_half; cc += 32) {
                const int col0 = half * ncol_half + cc;
                const int col = cb * N + col0;
                const long long my_off = (row < prm.rows && col < prm.cols) ? row_off + col : -1;
                const bool vec = (col + 32 <= prm.cols) && ((prm.cols & 3) == 0);
                // offsets of the 8 lines this lane will store, and their mask values, fetched before the
                // accumulator is even read so that the memory latency hides behind the TMEM load and the turn
                long long off[8];
                float4 mk[8];
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    off[rr] = __shfl_sync(0xffffffffu, my_off, 4 * rr + (lane >> 3));
                    mk[rr] = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (vec && use_mask && off[rr] >= 0) mk[rr] = __ldg(reinterpret_cast<const float4 *>(prm.mask + off[rr] + 4 * (lane & 7)));
                }
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
                        tma_store_3d(smem_u32(stg), &mapOut, col, rb1 * 128 + q * 32, (prm.direct ? 0 : split * 16) + t);
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
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_rank0(acce_bar(buf)));
            buf ^= 1;
        }
        // the last stores must have reached memory before the CTA ends
        if (prm.tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // Neither CTA may leave (or free its tensor memory) while the other can still read its shared memory through an MMA or
    // signal one of its barriers: both are past their last accumulator here
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

