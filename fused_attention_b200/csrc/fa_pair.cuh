// Fused attention forward at head_dim 128 on PAIRS of CTAs (tcgen05 cta_group::2).
//
// Same arithmetic, roles and hand-overs as fa_fwd_pipelined<128> (fa_kernels.cuh); what changes is who
// feeds and who issues the MMAs.  A cluster of two CTAs (the two SMs of one TPC) works on 512 query rows of
// one (batch, head): CTA r of the pair owns rows [256 r, 256 r + 256) as its two 128-row tiles, keeps their
// S, P and O in its own tensor memory and runs its own softmax and epilogue warps, exactly as before.  But
//   - every MMA is one instruction of M = 256 issued by a thread of the even CTA (the leader) for both:
//     tile i of the leader and tile i of its peer together.  Each CTA supplies its own 128 rows of A (its Q
//     tile from shared memory, its P from tensor memory) and HALF of B: of a K tile the 64 keys
//     [64 r, 64 r + 64), of a V tile the 64 head columns [64 r, 64 r + 64).  So a K/V tile crosses from L2
//     to the pair once instead of once per CTA, and an SM reads 6 KiB of shared-memory operands per
//     128x128x16 MMA instead of 8: the Q K^T products no longer run at the limit of shared-memory bandwidth;
//   - what the leader's issuing warps wait for (tiles landed, S read, P written, O read out) is counted on
//     barriers in the leader's shared memory, on which the peer's warps and TMA copies arrive through the
//     cluster's shared address space; what they announce (S complete, P V complete, ring slot and query
//     buffer free) is committed once to each CTA's own copy of the barrier;
//   - tensor memory is allocated and released by both CTAs together, and the two leave together (a cluster
//     barrier), because the peer's shared and tensor memory are operands of the leader's MMAs to the end.
// Every CTA loads its own tiles with plain TMA copies.  Work items are whole (no divided last round): the
// launcher takes this kernel only for such calls.
// With a mask (kHasMask; rows of the mask must start on 16-byte boundaries) each CTA also brings in, by TMA
// and on barriers of its own, the 128 x 128 mask tile of each of its query tiles and every key step, into
// one buffer per query tile; the softmax threads add their row of it to the scores and hand the buffer
// back at once, so the next step's tile is on its way while this step's exponentials are taken.  The ring
// is shorter to make room for the two buffers.
#pragma once

#include "fa_kernels.cuh"

namespace fa {

template <bool kHasMask = false>
struct PairCfgT {
    static constexpr int H = 128;
    using G = TileGeom<128>;
    static constexpr int kSlots = kHasMask ? 4 : 8;         // ring slots of HALF a K or V tile each
    static constexpr int kSlotBytes = G::kTileBytes / 2;    // 16 KiB: 64 keys x 128 columns, or 128 keys x 64 columns
    static constexpr int kQBytes = 2 * G::kTileBytes;       // this CTA's two query tiles
    static constexpr int kRingBytes = kSlots * kSlotBytes;
    static constexpr int kMaskTileBytes = kTile * kTile * 2;            // 128 x 128 fp16: two boxes of 64 keys
    static constexpr int kMaskBytes = kHasMask ? 2 * kMaskTileBytes : 0;   // one buffer per query tile
    static constexpr int kStageBytes = 4 * 32 * 128;        // epilogue staging: per warp 32 rows x 64 fp16
    static constexpr int kSmemBytes = kQBytes + kRingBytes + kMaskBytes + kStageBytes + 1024;   // + alignment slack
    static constexpr uint32_t kTmemCols = 512;
    // tensor memory columns, in each CTA: S [0,128) shared by its two tiles in turn, P0 [128,192), P1 [192,256),
    // O0 [256,384), O1 [384,512)
    static constexpr uint32_t kColS = 0, kColP0 = 128, kColP1 = 192, kColO0 = 256, kColO1 = 384;
    static constexpr int kHeldChunks = 1;
};
using PairCfg = PairCfgT<false>;

// S[256 x 128] = Q[256 x 128] K[128 x 128]^T for tile i of both CTAs: A = this CTA's Q tile (two boxes of
// 128 rows x 64 columns), B = this CTA's half of the K tile (two boxes of 64 keys x 64 columns).
__device__ __forceinline__ void issue_qk_pair(uint32_t tS, uint32_t sQ, uint32_t sKhalf) {
    constexpr uint32_t idesc = make_idesc_f16_pair(kTile, 0);
    const uint64_t dq = make_smem_desc<128>(sQ, 16), dk = make_smem_desc<128>(sKhalf, 16);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t box = (ks * 16) / 64, in_box = ((ks * 16) % 64) * 2;
        const uint32_t off_q = box * (kTile * 128) + in_box;         // 16 KiB per box of 128 rows
        const uint32_t off_k = box * ((kTile / 2) * 128) + in_box;   // 8 KiB per box of 64 rows
        mma_ss_pair(tS, dq + (off_q >> 4), dk + (off_k >> 4), idesc, ks > 0 ? 1u : 0u);
    }
}

// O[256 x 128] (+)= P[256 x 128] V[128 x 128]: A = this CTA's P (fp16 in tensor memory), B = this CTA's 64
// head columns of the V tile (one box of 128 keys x 64 columns, MN-major).
__device__ __forceinline__ void issue_pv_pair(uint32_t tO, uint32_t tP, uint32_t sVhalf, uint32_t accumulate) {
    constexpr uint32_t idesc = make_idesc_f16_pair(128, 1);
    const uint64_t dv = make_smem_desc<128>(sVhalf, PairCfg::kSlotBytes);   // (the same in both instances)
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
        mma_ts_pair(tO, tP + ks * 8, dv + ((ks * 16 * 128) >> 4), idesc, (accumulate | ks) ? 1u : 0u);
}

// grid = 2 * min(pairs of SMs, work items), clusters of 2, block = 512.  A work item is 512 query rows of one
// (batch, head): n_items = ceil(L / 512) * R * B, numbered row-block fastest; cluster c takes items c,
// c + clusters, ...  Warp roles as in fa_fwd_pipelined<128>; in the peer CTA the two issuing warps only
// take part in allocating and releasing tensor memory.
// tmM is the map of the mask (boxes of 128 rows x 64 keys); instances without a mask get any valid map.
template <bool kHasMask>
__global__ void __launch_bounds__(512, 1)
fa_fwd_pair(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKh,
            const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmY,
            const __grid_constant__ CUtensorMap tmM, const Params p) {
    constexpr int H = 128;
    using G = TileGeom<128>;
    using C = PairCfgT<kHasMask>;
    constexpr int NS = C::kSlots;
    enum {
        BAR_QFULL0 = 0, BAR_QFULL1,  // leader: query tile i of both CTAs landed (bytes of both)
        BAR_QEMPTY0, BAR_QEMPTY1,    // each CTA: the item's last Q K^T of tile i has retired
        BAR_S0, BAR_S1,              // each CTA: S of tile i complete
        BAR_P0, BAR_P1,              // leader: P of tile i written in both CTAs (8 warps)
        BAR_SFREE,                   // leader: S read into registers in both CTAs (8 warps), one phase per use
        BAR_PV0, BAR_PV1,            // each CTA: P V of tile i complete
        BAR_A0, BAR_A1,              // each CTA: final row sums of tile i in shared memory (4 warps)
        BAR_OFREE0, BAR_OFREE1,      // leader: O of tile i read out in both CTAs (8 warps)
        BAR_OLOCAL0, BAR_OLOCAL1,    // each CTA: O of tile i read out here (4 warps), for its softmax warps
        BAR_FINAL, BAR_FINAL2,       // leader: every MMA of an issuing warp retired
        BAR_MFULL0, BAR_MFULL1,      // each CTA: the mask tile of its query tile i and this key step landed
        BAR_MEMPTY0, BAR_MEMPTY1,    // each CTA: that tile has been read by the 4 softmax warps of tile i
        BAR_FULL,                    // leader: NS ring barriers, both halves of a tile landed
        BAR_EMPTY = BAR_FULL + NS,   // each CTA: NS ring barriers, slot free
        BAR_COUNT = BAR_EMPTY + NS
    };

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[BAR_COUNT];
    __shared__ float l_buf[2][2][kTile];  // [item parity][tile][row] final row sums
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;

    const uint32_t tid = threadIdx.x;
#ifdef FA_CYCLES
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) p.cycles[4 * (p.launch_id & 63u)] = global_timer_ns();
#endif
    const uint32_t warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t lane = tid & 31u;
    const uint32_t rank = cluster_cta_rank();          // 0 = leader
    const uint32_t cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const uint32_t n = p.n_kv_tiles;
    const uint32_t q_quads = (p.q_pairs + 1u) >> 1;     // blocks of 512 query rows per (batch, head)
    const uint32_t n_items = q_quads * p.R * p.B;
    const uint32_t my_items = cluster < n_items ? (n_items - cluster + n_clusters - 1u) / n_clusters : 0u;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base;                   // two tiles
    const uint32_t sRing = smem_base + C::kQBytes;   // NS half tiles
    const uint32_t sMask = sRing + C::kRingBytes;    // two mask tiles (instance with a mask only)
    const uint32_t sStage = sMask + C::kMaskBytes;   // epilogue staging, 4 KiB per epilogue warp
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };                                   // this CTA's copy
    const uint32_t bar0_leader = map_to_cta(bar0, 0), bar0_peer = map_to_cta(bar0, 1);
    auto lbar = [&](int i) { return bar0_leader + 8u * i; };                           // the leader's copy (cluster address)
    const WaitCtl ctl{p.status, &abort_flag, kWaitCapCycles, p.status + 2, p.launch_id};

    if (tid == 0) {
        prefetch_tensormap(&tmY);
#pragma unroll
        for (int i = 0; i < BAR_COUNT; ++i) {
            uint32_t count = 1;
            if (i == BAR_P0 || i == BAR_P1 || i == BAR_SFREE || i == BAR_OFREE0 || i == BAR_OFREE1) count = 8;
            if (i == BAR_A0 || i == BAR_A1 || i == BAR_OLOCAL0 || i == BAR_OLOCAL1 || i == BAR_MEMPTY0 || i == BAR_MEMPTY1) count = 4;
            mbar_init(bar(i), count);
        }
        abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmKh);
        prefetch_tensormap(&tmV);
        if constexpr (kHasMask) prefetch_tensormap(&tmM);
    }
#ifdef FA_DEBUG
    dbg_begin(p, ctl, smem_base, C::kSmemBytes - 1024);
#endif
    if (warp == 12) {
        tmem_alloc_pair(smem_u32(&tmem_slot), C::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
#ifdef FA_DEBUG
    if (tid == 0) dbg_tmem(tmem_slot, C::kTmemCols);
#endif
    // both CTAs have their barriers and their tensor memory before either signals or multiplies anything
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    grid_dep_wait();
    grid_dep_launch();
    if (tid == 15 * 32) leave_early_if_launch_failed(ctl);
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
#ifdef FA_CYCLES
    long long cyc0 = 0;
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) {
        p.cycles[4 * (p.launch_id & 63u) + 1] = global_timer_ns();
        cyc0 = clock64();
    }
#endif

    if (warp < 8) {
        // ------------------------------------------------------------------ softmax, tile i of this CTA
        setmaxnreg_inc<184>();
        const uint32_t i = warp >> 2;
        const uint32_t row = tid & 127u;
        const uint32_t lane_off = ((warp & 3u) * 32u) << 16;
        const uint32_t tS = tmem_base + lane_off + C::kColS;
        const uint32_t tP = tmem_base + lane_off + (i ? C::kColP1 : C::kColP0);
        const uint32_t tO = tmem_base + lane_off + (i ? C::kColO1 : C::kColO0);
        const float c = p.scale_log2;
        uint32_t g = 0;   // global step
        float l_last = 1.f;
        for (uint32_t k = 0; k < my_items; ++k) {
            float m = -INFINITY, l = 0.f;
            for (uint32_t j = 0; j < n; ++j, ++g) {
                // (time line, softmax warp of rows 0-31: 0 looks for S, 1 S there, 2 S in registers, 3 first 32
                // exponentials taken, 4 P buffer free, 5 all exponentials taken and P stored, 6 P handed over)
                if ((warp & 3u) == 0u) FA_STAMP(i, g, 0);
                mbar_wait(bar(BAR_S0 + i), g & 1u, ctl, kRoleSoftmax | (BAR_S0 + i));
                if ((warp & 3u) == 0u) FA_STAMP(i, g, 1);
                tc_fence_after();
                __syncwarp();
                float s[kTile];
                const bool ragged = (j + 1) * kTile > p.L;
                const bool first = j == 0;
                load_s_row(tS, s);
                if ((warp & 3u) == 0u) FA_STAMP(i, g, 2);
                // S is in registers: the leader may overwrite it (in both CTAs) with the next scores
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lbar(BAR_SFREE));
                if constexpr (kHasMask) {
                    // this tile's mask tile of this step; its buffer is handed back as soon as it has been read
                    mbar_wait(bar(BAR_MFULL0 + i), g & 1u, ctl, kRoleSoftmax | (BAR_MFULL0 + i));
                    add_mask_tile_row(s, sMask + i * C::kMaskTileBytes, row, p.mask_to_score);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(BAR_MEMPTY0 + i));
                }
                if (ragged) mask_tail(s, static_cast<int>(p.L - j * kTile));
                if (first) m = row_max(s);
                {
                    // A row that has seen nothing but -inf so far (possible only with a mask) takes 0 as the
                    // reference of its exponents, so that P = 0 and l = 0 instead of inf - inf.
                    float nmc = -m * c;
                    if constexpr (kHasMask) nmc = (m == -INFINITY) ? 0.f : nmc;
                    float mx4[4];   // (not used: the row maximum is only taken when the row sum asks for it)
                    uint32_t held[16 * C::kHeldChunks];
                    float sum = exp_chunks<0, C::kHeldChunks, false, false>(s, c, nmc, tP, mx4, held);
                    if ((warp & 3u) == 0u) FA_STAMP(i, g, 3);
                    if (g > 0) {
                        mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                        tc_fence_after();
                    }
                    if ((warp & 3u) == 0u) FA_STAMP(i, g, 4);
#pragma unroll
                    for (int ch = 0; ch < C::kHeldChunks; ++ch) tmem_st16(tP + ch * 16, held + ch * 16);
                    sum += exp_chunks<C::kHeldChunks, 4, false>(s, c, nmc, tP, mx4);
                    if ((warp & 3u) == 0u) FA_STAMP(i, g, 5);
                    // The reference has to move when a score exceeds it by more than 2^8 in the exp2 domain, that is
                    // when a P exceeds 2^8.  No P can while the row's sum of P stays below 2^8, so the row maximum is
                    // only taken in a warp where some row's sum says it might (the same decisions as testing every
                    // row's maximum, which is what costs 64 instructions per row and step).
                    float mx = m;
                    bool moved = false;
                    if (__any_sync(0xffffffffu, sum > kLazyRescaleSum)) {
                        mx = row_max(s);
                        moved = (mx - m) * c > kLazyRescaleLog2;
                    }
                    if (__any_sync(0xffffffffu, moved)) {
                        const float m_new = moved ? mx : m;
                        const float alpha = moved ? ex2_approx((m - m_new) * c) : 1.f;
                        m = m_new;
                        float nmc2 = -m * c;
                        if constexpr (kHasMask) nmc2 = (m == -INFINITY) ? 0.f : nmc2;
                        float unused[4];
                        l = l * alpha + exp_chunks<0, 4, false>(s, c, nmc2, tP, unused);
                        if (g > 0) mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                        tc_fence_after();
                        __syncwarp();
                        if (!first) rescale_o_row<H>(tO, alpha);
                    } else {
                        l += sum;
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lbar(BAR_P0 + i));
                if ((warp & 3u) == 0u) FA_STAMP(i, g, 6);
            }
            l_last = l;
            if (k + 1u < my_items) {   // (the CTA's last item: see below)
                if (k > 0) mbar_wait(bar(BAR_OLOCAL0 + i), (k - 1u) & 1u, ctl, kRoleSoftmax | (BAR_OLOCAL0 + i));
                l_buf[k & 1u][i][row] = l;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_A0 + i));
            }
        }
        if (my_items > 0u) {
            // The CTA's last item: nothing is left to overlap its epilogue with, so the softmax warps write Y
            // themselves, both tiles at once (each thread has its row sum, and the registers to take the whole O row
            // in one round trip), instead of handing the two tiles to the four epilogue warps one after the other.
            // Staging area: the tile's own query buffer, which its last Q K^T has long let go of; 8 KiB per warp.
            const uint32_t item = cluster + (my_items - 1u) * n_clusters;
            const uint32_t q_quad = item % q_quads, bh = item / q_quads;
            const uint32_t wq = warp & 3u;
            const int32_t row0 = static_cast<int32_t>(((q_quad * 2u + rank) * 2u + i) * kTile + wq * 32u);
            const uint32_t stage = sQ + i * G::kTileBytes + wq * 8192u;
            mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
            tc_fence_after();
            __syncwarp();
            stage_o_row<H>(tO, 1.f / l_last, stage, lane);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < static_cast<int32_t>(p.L)) {
#pragma unroll
                for (int half = 0; half < H / 64; ++half)
                    tma_store_3d(&tmY, stage + half * 4096u, static_cast<int32_t>((bh % p.R) * H + half * 64), row0,
                                 static_cast<int32_t>(bh / p.R));
                bulk_commit_group();
            }
            if (lane == 0) bulk_wait_read_all();   // the staging area is this CTA's until TMA has read it
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ epilogue: Y = O / l, this CTA's tiles
        setmaxnreg_dec<64>();
        const uint32_t row = tid & 127u;
        const uint32_t wq = warp & 3u;
        const uint32_t lane_off = (wq * 32u) << 16;
        const uint32_t stage = sStage + wq * 4096u;
        uint32_t k = 0;
        // (the CTA's last item is written by the softmax warps)
        for (uint32_t item = cluster; k + 1u < my_items; item += n_clusters, ++k) {
            const uint32_t q_quad = item % q_quads, bh = item / q_quads;
            const uint32_t head = bh % p.R, batch = bh / p.R;
#pragma unroll
            for (uint32_t i = 0; i < 2; ++i) {
                mbar_wait_relaxed(bar(BAR_A0 + i), k & 1u, ctl, kRoleEpilogue | (BAR_A0 + i), 100);
                const float inv_l = 1.f / l_buf[k & 1u][i][row];
                mbar_wait(bar(BAR_PV0 + i), (k * n + n - 1u) & 1u, ctl, kRoleEpilogue | (BAR_PV0 + i));
                tc_fence_after();
                __syncwarp();
                const uint32_t tO = tmem_base + lane_off + (i ? C::kColO1 : C::kColO0);
                const int32_t row0 = static_cast<int32_t>(((q_quad * 2u + rank) * 2u + i) * kTile + wq * 32u);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (lane == 0) bulk_wait_read_all();
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float o[16];
                        tmem_ld16(tO + half * 64 + c * 16, o);
                        tmem_wait_ld();
                        if (half == 1 && c == 3) {
                            // the whole O tile has left tensor memory: the leader may overwrite it, and this
                            // CTA's softmax warps may hand over the next item's row sums
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) {
                                mbar_arrive_cluster(lbar(BAR_OFREE0 + i));
                                mbar_arrive(bar(BAR_OLOCAL0 + i));
                            }
                        }
#pragma unroll
                        for (int v4 = 0; v4 < 2; ++v4) {
                            const uint32_t w0 = pack_half2(o[v4 * 8 + 0] * inv_l, o[v4 * 8 + 1] * inv_l);
                            const uint32_t w1 = pack_half2(o[v4 * 8 + 2] * inv_l, o[v4 * 8 + 3] * inv_l);
                            const uint32_t w2 = pack_half2(o[v4 * 8 + 4] * inv_l, o[v4 * 8 + 5] * inv_l);
                            const uint32_t w3 = pack_half2(o[v4 * 8 + 6] * inv_l, o[v4 * 8 + 7] * inv_l);
                            const uint32_t chunk = static_cast<uint32_t>(c * 2 + v4) ^ (lane & 7u);
                            st_shared_v4(stage + lane * 128u + chunk * 16u, w0, w1, w2, w3);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < static_cast<int32_t>(p.L)) {
                        tma_store_3d(&tmY, stage, static_cast<int32_t>(head * H + half * 64), row0,
                                     static_cast<int32_t>(batch));
                        bulk_commit_group();
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_read_all();
    } else {
        setmaxnreg_dec<80>();
        if ((warp == 12 || warp == 14) && rank == 0) {
            // -------------------------------------------------------------- MMA issue (leader only)
            const bool leader = elect_one();
            const uint32_t tS = tmem_base + C::kColS;
            const uint32_t tO0 = tmem_base + C::kColO0, tO1 = tmem_base + C::kColO1;
            const uint32_t tP0 = tmem_base + C::kColP0, tP1 = tmem_base + C::kColP1;
            auto slot_addr = [&](uint32_t t) { return sRing + (t % NS) * C::kSlotBytes; };
            bool ok = true;
            auto mwait = [&](int b, uint32_t parity) { ok &= mbar_wait(bar(b), parity, ctl, kRoleMma | static_cast<uint32_t>(b)); };
            auto wait_full = [&](uint32_t t) { mwait(BAR_FULL + (t % NS), (t / NS) & 1u); };
            // one arrival on this barrier in the leader and one on its copy in the peer when the MMAs issued so far are done
            auto commit_both = [&](int b) {
                tc_commit_pair(bar0_leader + 8u * b);
                tc_commit_pair(bar0_peer + 8u * b);
            };
            const uint32_t steps = my_items * n;
            // ring item 2g is the K tile of global step g, item 2g+1 its V tile (each CTA holds its half)
            mbar_poll_declare();
            if (warp == 12) {
                // Q K^T stream.  Uses of the one S buffer are numbered 2g + i; use u needs use u - 1 to have been read.
                bool polled = false;
                uint32_t k = 0, j = 0;
                for (uint32_t g = 0; g < steps; ++g) {
                    const bool new_item = j == 0;
                    const bool last_of_item = j + 1 == n;
                    const uint32_t tk = 2 * g;
                    // (time line: 0 top of the step, 1 K and Q there, 2 S buffer read by tile 1: tile 0's Q K^T goes
                    // out, 3 issued, 4 S buffer read by tile 0: tile 1's Q K^T goes out, 5 issued)
                    FA_STAMP(2u, g, 0);
                    if (!(polled && mbar_poll_end<0>())) wait_full(tk);
                    if (new_item) mwait(BAR_QFULL0, k & 1u);
                    FA_STAMP(2u, g, 1);
                    if (g > 0) mwait(BAR_SFREE, 1u);
                    FA_STAMP(2u, g, 2);
                    tc_fence_after();
                    if (leader && ok) {
                        issue_qk_pair(tS, sQ, slot_addr(tk));
                        commit_both(BAR_S0);
                        if (last_of_item) commit_both(BAR_QEMPTY0);
                    }
                    FA_STAMP(2u, g, 3);
                    if (new_item) mwait(BAR_QFULL1, k & 1u);
                    mwait(BAR_SFREE, 0u);
                    FA_STAMP(2u, g, 4);
                    tc_fence_after();
                    polled = g + 1 < steps;
                    if (polled) {
                        const uint32_t nk = tk + 2;
                        mbar_poll_begin<0>(bar(BAR_FULL + (nk % NS)), (nk / NS) & 1u);
                    }
                    if (leader && ok) {
                        issue_qk_pair(tS, sQ + G::kTileBytes, slot_addr(tk));
                        commit_both(BAR_S1);
                        if (last_of_item) commit_both(BAR_QEMPTY1);
                        commit_both(BAR_EMPTY + (tk % NS));
                    }
                    FA_STAMP(2u, g, 5);
                    if (++j == n) { j = 0; ++k; }
                }
            } else {
                // P V stream
                bool polled = false;
                uint32_t k = 0, j = 0;
                for (uint32_t g = 0; g < steps; ++g) {
                    const uint32_t tv = 2 * g + 1;
                    const uint32_t acc = j > 0 ? 1u : 0u;
                    // (time line: 0 top of the step, 1 V there and O free, 2 P of tile 0 there: its P V goes out,
                    // 3 issued, 4 P of tile 1 there: its P V goes out, 5 issued)
                    FA_STAMP(3u, g, 0);
                    if (!(polled && mbar_poll_end<1>())) wait_full(tv);
                    if (j == 0 && k > 0) mwait(BAR_OFREE0, (k - 1u) & 1u);
                    FA_STAMP(3u, g, 1);
                    mwait(BAR_P0, g & 1u);
                    FA_STAMP(3u, g, 2);
                    tc_fence_after();
                    if (leader && ok) {
                        issue_pv_pair(tO0, tP0, slot_addr(tv), acc);
                        commit_both(BAR_PV0);
                    }
                    FA_STAMP(3u, g, 3);
                    if (j == 0 && k > 0) mwait(BAR_OFREE1, (k - 1u) & 1u);
                    mwait(BAR_P1, g & 1u);
                    FA_STAMP(3u, g, 4);
                    tc_fence_after();
                    polled = g + 1 < steps;
                    if (polled) {
                        const uint32_t nv = tv + 2;
                        mbar_poll_begin<1>(bar(BAR_FULL + (nv % NS)), (nv / NS) & 1u);
                    }
                    if (leader && ok) {
                        issue_pv_pair(tO1, tP1, slot_addr(tv), acc);
                        commit_both(BAR_PV1);
                        commit_both(BAR_EMPTY + (tv % NS));
                    }
                    FA_STAMP(3u, g, 5);
                    if (++j == n) { j = 0; ++k; }
                }
            }
            // every MMA this warp issued has retired (in both CTAs) before either CTA releases anything
            const int bar_final = warp == 12 ? BAR_FINAL : BAR_FINAL2;
            if (leader) tc_commit_pair(bar0_leader + 8u * bar_final);
            __syncwarp();
            mbar_wait_certain(bar(bar_final), 0, ctl, kRoleMma | static_cast<uint32_t>(bar_final));
        } else if (warp == 13 && elect_one()) {
            // -------------------------------------------------------------- TMA producer (both CTAs)
            // Each CTA copies its own query tiles and its own half of every K and V tile into its own shared
            // memory; the bytes are counted on the leader's barrier, which expects both CTAs' shares.
            uint32_t t = 0, k = 0;
            bool stop = false;
            bool q_pending[2] = {false, false};
            for (uint32_t item = cluster; item < n_items && !stop; item += n_clusters, ++k) {
                const uint32_t q_quad = item % q_quads, bh = item / q_quads;
                const int32_t col0 = static_cast<int32_t>((bh % p.R) * H);
                const int32_t batch = static_cast<int32_t>(bh / p.R);
                const int32_t q_row0 = static_cast<int32_t>((q_quad * 2u + rank) * 2u * kTile);
                for (uint32_t tt = 0; tt < 2 * n; ++tt, ++t) {
                    if (tt < 2) {
                        if (k > 0 && !mbar_wait(bar(BAR_QEMPTY0 + tt), (k - 1u) & 1u, ctl,
                                                kRoleProducer | (BAR_QEMPTY0 + tt))) { stop = true; break; }
                        if (rank == 0) mbar_expect_tx(bar(BAR_QFULL0 + tt), 2 * G::kTileBytes);
                        const uint32_t dst = sQ + tt * G::kTileBytes;
                        const int32_t r0 = q_row0 + static_cast<int32_t>(tt * kTile);
                        tma_load_3d_pair(dst, &tmQ, lbar(BAR_QFULL0 + tt), col0, r0, batch);
                        tma_load_3d_pair(dst + G::kBoxBytes, &tmQ, lbar(BAR_QFULL0 + tt), col0 + 64, r0, batch);
                        q_pending[tt] = true;
                    }
                    const uint32_t slot = t % NS;
                    if (!mbar_wait(bar(BAR_EMPTY + slot), ((t / NS) & 1u) ^ 1u, ctl,
                                   kRoleProducer | (BAR_EMPTY + slot))) { stop = true; break; }
                    if (rank == 0) mbar_expect_tx(bar(BAR_FULL + slot), 2 * C::kSlotBytes);
                    const uint32_t dst = sRing + slot * C::kSlotBytes;
                    const int32_t key0 = static_cast<int32_t>((tt >> 1) * kTile);
                    if ((tt & 1u) == 0) {
                        // K: this CTA's 64 keys, all 128 columns (two boxes of 64 x 64)
                        const int32_t r0 = key0 + static_cast<int32_t>(rank * 64u);
                        tma_load_3d_pair(dst, &tmKh, lbar(BAR_FULL + slot), col0, r0, batch);
                        tma_load_3d_pair(dst + C::kSlotBytes / 2, &tmKh, lbar(BAR_FULL + slot), col0 + 64, r0, batch);
                    } else {
                        // V: all 128 keys, this CTA's 64 columns (one box of 128 x 64)
                        tma_load_3d_pair(dst, &tmV, lbar(BAR_FULL + slot), col0 + static_cast<int32_t>(rank * 64u), key0, batch);
                    }
                }
            }
            if (abort_flag != 0u && (q_pending[0] || q_pending[1] || t > 0u)) {
                // A wait gave up.  This CTA's last copies may still be landing in its shared memory and their
                // barrier lives in the leader, where the peer cannot poll it: give them a bounded time
                // (hundreds of times a copy's latency) before the CTA goes on to leave.
                for (int spin = 0; spin < 200; ++spin) __nanosleep(1000);
            }
        } else if (kHasMask && warp == 15 && elect_one()) {
            // -------------------------------------------------------------- TMA producer of the mask tiles (both CTAs)
            // Tile i's buffer is filled for key step g as soon as the tile's softmax warps have read step g - 1
            // out of it.  Boxes that lie beyond the end of the sequence (keys or rows) arrive as zeros.
            uint32_t g = 0;   // global step
            uint32_t asked[2] = {0, 0};   // for how many key steps tile i's mask tile has been asked for
            bool stop = false;
            for (uint32_t item = cluster; item < n_items && !stop; item += n_clusters) {
                const uint32_t q_quad = item % q_quads, bh = item / q_quads;
                const int32_t batch = static_cast<int32_t>(bh / p.R);
                const int32_t q_row0 = static_cast<int32_t>((q_quad * 2u + rank) * 2u * kTile);
                for (uint32_t j = 0; j < n && !stop; ++j, ++g) {
                    const int32_t key0 = static_cast<int32_t>(j * kTile);
                    for (uint32_t i = 0; i < 2; ++i) {
                        if (g > 0 && !mbar_wait(bar(BAR_MEMPTY0 + i), (g - 1u) & 1u, ctl, kRoleProducer | (BAR_MEMPTY0 + i))) {
                            stop = true;
                            break;
                        }
                        const uint32_t dst = sMask + i * C::kMaskTileBytes;
                        const int32_t r0 = q_row0 + static_cast<int32_t>(i * kTile);
                        mbar_expect_tx(bar(BAR_MFULL0 + i), C::kMaskTileBytes);
                        tma_load_3d(dst, &tmM, bar(BAR_MFULL0 + i), key0, r0, batch);
                        tma_load_3d(dst + kTile * 128, &tmM, bar(BAR_MFULL0 + i), key0 + 64, r0, batch);
                        asked[i] = g + 1u;
                    }
                }
            }
            if (abort_flag != 0u) {   // do not leave while the mask tiles asked for last may still be landing
                for (uint32_t i = 0; i < 2; ++i) {
                    const long long t_0 = clock64();
                    while (asked[i] > 0u && !mbar_try_wait(bar(BAR_MFULL0 + i), (asked[i] - 1u) & 1u) &&
                           clock64() - t_0 < 200000000LL) {
                    }
                }
            }
        }
    }

    // Nothing is released, and neither CTA leaves, before both are through: until the leader's last MMA has
    // retired the peer's shared and tensor memory are its operands, and until the peer's last arrival the
    // leader's barriers are its targets.
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
#ifdef FA_CYCLES
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) {
        p.cycles[4 * (p.launch_id & 63u) + 2] = global_timer_ns();
        p.cycles[4 * (p.launch_id & 63u) + 3] = static_cast<unsigned long long>(clock64() - cyc0);
    }
#endif
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

}  // namespace fa
