// Fused multi-head attention forward for sm_100a:  Y = softmax(Q K^T / sqrt(H)) V.
//
// Two kernels share the same arithmetic:
//   fa_fwd_simple<H, kHasMask>  one 128-row query tile per CTA, 128 threads, every step in program
//                               order.  Covers every head_dim (16, 32, 64, 128), the additive mask
//                               and tiny problems; several CTAs per SM overlap one another.
//   fa_fwd_pipelined<H>         two 128-row query tiles per CTA, 512 threads split into roles
//                               (2 softmax warpgroups, 1 epilogue warpgroup, 1 MMA warp, 1 TMA
//                               warp); K/V stream through a shared-memory ring; the softmax of one
//                               tile overlaps the MMAs of the other.  H in {64, 128}, no mask.
//
// What they replace in the reference (include/fused_attn.cuh): attention_kernel (605-858) and the
// threadblock_* primitives it calls (48-521).  The maths is the reference's blockwise merge of
// (row max, row sum, numerator) (458-521; README.md:45-61) with these deliberate differences:
// fp32 scores, running max, running sum and numerator (the reference keeps all of them in fp16),
// exp2 with log2(e)/sqrt(H) folded into one multiply-add, and key tiles that may be ragged.
//
// Data layout.  Q, K, V, Y: [B, L, F] fp16, head h in columns [h*H, (h+1)*H).  A TMA tensor map
// sees each input as a 3-D tensor {F, L, B}; a tile is 128 rows x H columns fetched as H/64 boxes
// of 128 x 64 (one box of 128 x H for H < 64) with the swizzle span equal to the box row, so a box
// lands in shared memory as 128 rows of 128 (64, 32) bytes.  Rows beyond L are zero-filled by TMA.
// That layout is the canonical K-major operand (Q and K for S = Q K^T) and, read with the
// MN-major bit set, the canonical operand for V in O = P V, so V is never transposed.
//
// TMEM (columns of 128 lanes x 32 bit): S tile 128 columns of fp32; P (fp16, two per column) 64
// columns; O tile H columns of fp32.  In the simple kernel P overwrites the first 64 columns of
// its S; in the pipelined kernel P has columns of its own (PipeCfg).
#pragma once

#include <cuda.h>
#include "fa_ptx.cuh"

namespace fa {

struct Params {
    __half* y;            // [B, L, F]
    const __half* mask;   // [B, L, L] or nullptr
    uint32_t* status;     // device status block {code, count, launch id, -}, see WaitCtl
    uint32_t launch_id;   // non-zero and different for every launch of the process
    uint32_t n_q_tiles;   // ceil(L / 128)
    uint32_t B, L, F;
    uint32_t n_kv_tiles;  // ceil(L / 128)
    uint32_t R;           // heads = F / H
    uint32_t q_pairs;     // ceil(L / 256): pairs of query tiles per (batch, head)
    uint32_t n_items;     // q_pairs * R * B: work items of the pipelined kernel
    float scale_log2;     // log2(e) / sqrt(H)
    float mask_to_score;  // sqrt(H): mask value m enters as s + m*sqrt(H) before the folded scale
#if defined(FA_TRACE) || defined(FA_CYCLES)
    unsigned long long* trace;  // [8 slots][512] (clock64 << 8 | tag) of one CTA, see FA_TRACE_EV
    uint32_t trace_cta;         // linear block index that records
#endif
};

// Compile with -DFA_TRACE to make one CTA of the pipelined kernel record a time line: every role
// (slot) appends clock64() with a tag at its hand-over points.  Off in normal builds.
#ifdef FA_TRACE
#define FA_TRACE_DECL                                                                              \
    uint32_t tr_n = 0;                                                                             \
    const bool tr_on = p.trace != nullptr &&                                                       \
        (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) == p.trace_cta;
#define FA_TRACE_EV(slot, tag)                                                                     \
    do {                                                                                           \
        if (tr_on && tr_n < 512) {                                                                 \
            p.trace[(slot) * 512 + tr_n] = (static_cast<unsigned long long>(clock64()) << 8) | (tag); \
            ++tr_n;                                                                                \
        }                                                                                          \
    } while (0)
#else
#define FA_TRACE_DECL
#define FA_TRACE_EV(slot, tag) do {} while (0)
#endif

constexpr int kTile = 128;  // rows of a query tile and of a key/value tile

// role << 8 | barrier id, written to the status word when a bounded wait expires
enum : uint32_t {
    kRoleSimple = 0x100u,
    kRoleProducer = 0x200u,
    kRoleMma = 0x300u,
    kRoleSoftmax = 0x400u,
    kRoleEpilogue = 0x500u,
    kRoleDrain = 0x600u
};

template <int H>
struct TileGeom {
    static constexpr int kBoxCols = H < 64 ? H : 64;           // columns per TMA box
    static constexpr int kBoxes = H / kBoxCols;                // boxes per tile
    static constexpr int kSwz = kBoxCols * 2;                  // swizzle span = row pitch, bytes
    static constexpr int kBoxBytes = kTile * kBoxCols * 2;     // 16 KiB at H >= 64
    static constexpr int kTileBytes = kTile * H * 2;
};

// One TMA tile (all its boxes) -> shared memory at `dst`, signalling `bar`.
template <int H>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                          int32_t col0, int32_t row0, int32_t batch) {
    using G = TileGeom<H>;
    mbar_expect_tx(bar, G::kTileBytes);
#pragma unroll
    for (int b = 0; b < G::kBoxes; ++b)
        tma_load_3d(dst + b * G::kBoxBytes, map, bar, col0 + b * G::kBoxCols, row0, batch);
}

// S[128 x 128] = Q[128 x H] * K[128 x H]^T, both operands K-major in shared memory.
template <int H>
__device__ __forceinline__ void issue_qk(uint32_t tS, uint32_t sQ, uint32_t sK) {
    using G = TileGeom<H>;
    constexpr uint32_t idesc = make_idesc_f16(kTile, 0);
    const uint64_t dq = make_smem_desc<G::kSwz>(sQ, 16), dk = make_smem_desc<G::kSwz>(sK, 16);
#pragma unroll
    for (int ks = 0; ks < H / 16; ++ks) {
        // the address field counts 16-byte units, so stepping along K is an add on the low word
        const uint32_t off = ((ks * 16) / G::kBoxCols) * G::kBoxBytes + ((ks * 16) % G::kBoxCols) * 2;
        mma_ss(tS, dq + (off >> 4), dk + (off >> 4), idesc, ks > 0 ? 1u : 0u);
    }
}

// O[128 x H] (+)= P[128 x 128] * V[128 x H]; P is fp16 in TMEM, V is MN-major in shared memory.
// Issues the k-steps [kK0, kK1) of the eight (16 keys each), so that the product can start on the
// part of P that is already written.
template <int H, int kK0 = 0, int kK1 = kTile / 16>
__device__ __forceinline__ void issue_pv(uint32_t tO, uint32_t tP, uint32_t sV, uint32_t accumulate) {
    using G = TileGeom<H>;
    constexpr uint32_t idesc = make_idesc_f16(H, 1);
    const uint64_t dv = make_smem_desc<G::kSwz>(sV, G::kBoxBytes);
#pragma unroll
    for (int ks = kK0; ks < kK1; ++ks) {
        // 16 key rows per step: 8 TMEM columns of packed fp16 pairs, 16 shared-memory rows.
        mma_ts(tO, tP + ks * 8, dv + ((ks * 16 * G::kSwz) >> 4), idesc, (accumulate | ks) ? 1u : 0u);
    }
}

// Maximum of one score row (3-input max: two elements per instruction, four chains).
__device__ __forceinline__ float row_max(const float (&s)[kTile]) {
    float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
    float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
    for (int i = 12; i + 8 <= kTile; i += 8) {
        mx0 = max3(mx0, s[i], s[i + 1]);
        mx1 = max3(mx1, s[i + 2], s[i + 3]);
        mx2 = max3(mx2, s[i + 4], s[i + 5]);
        mx3 = max3(mx3, s[i + 6], s[i + 7]);
    }
    // 12 + 8*14 = 124: four elements left
    mx0 = max3(mx0, s[124], s[125]);
    mx1 = max3(mx1, s[126], s[127]);
    return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

// Running-maximum update of the online softmax.
//   m      reference maximum that the exponents are taken against (updated)
//   mx     maximum of the new score row;  c  log2(e)/sqrt(H)
// Returns alpha, the factor by which everything accumulated before this step must be multiplied,
// and nmc = -m*c, the addend of the folded exponent s*c - m*c.
// The reference maximum only moves when the new row exceeds it by more than 2^8 in the exp2
// domain: P then stays below 256 (exact in fp16 to 11 bits like any other magnitude), sum and
// numerator are fp32, and alpha is exactly 1 on most steps, which lets the O rescale be skipped.
// The final Y = O / l does not depend on which reference was used.
constexpr float kLazyRescaleLog2 = 8.f;
__device__ __forceinline__ float update_max(float& m, const float mx, const float c, float& nmc) {
    const float m_new = fmaxf(m, mx);
    const bool keep = (m_new - m) * c <= kLazyRescaleLog2;   // false for the first tile (m = -inf)
    // A row that has seen nothing but -inf so far (possible only with an additive mask) uses 0
    // as its reference, so that p = 0 and l = 0 instead of inf - inf.
    const float m_use = keep ? m : ((m_new == -INFINITY) ? 0.f : m_new);
    const float alpha = keep ? 1.f : ex2_approx((m - m_use) * c);
    nmc = -m_use * c;
    m = keep ? m : m_new;
    return alpha;
}

// P = exp2(s*c + nmc) for one whole score row: written as fp16 into 64 TMEM columns at tP (two values
// per column, even key index in the low half); returns the fp32 row sum of P.
__device__ __forceinline__ float exp_and_store_p(const float (&s)[kTile], const float c,
                                                 const float nmc, const uint32_t tP) {
    const uint64_t c2 = pack_f32x2(c, c), n2 = pack_f32x2(nmc, nmc);
    uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(s[chunk * 32 + 2 * e], s[chunk * 32 + 2 * e + 1]), c2, n2), x0, x1);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            if (e & 1) sum_b = add_f32x2(sum_b, pack_f32x2(p0, p1));
            else sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
            pk[e] = pack_half2(p0, p1);
        }
        tmem_st16(tP + chunk * 16, pk);
    }
    float lo, hi;
    unpack_f32x2(add_f32x2(sum_a, sum_b), lo, hi);
    return lo + hi;
}

// P = exp2(s*c + nmc) for the 32-key chunks [kC0, kC1) of one score row, written as fp16 into TMEM
// at tP + 16*chunk (two values per column, even key index in the low half); returns the fp32 sum of
// those P.  With kWithMax the running maxima mx[] take in the scores of these chunks in the same
// pass (the maximum instructions fill the issue slots the MUFU leaves free).
// With kStore false the packed P are not written to TMEM but handed back in pk_out (16 words per
// chunk), for the caller to store once the P buffer is free.
template <int kC0, int kC1, bool kWithMax, bool kStore = true>
__device__ __forceinline__ float exp_chunks(const float (&s)[kTile], const float c, const float nmc,
                                            const uint32_t tP, float (&mx)[4], uint32_t* pk_out = nullptr) {
    const uint64_t c2 = pack_f32x2(c, c), n2 = pack_f32x2(nmc, nmc);
    uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
    for (int chunk = kC0; chunk < kC1; ++chunk) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float s0 = s[chunk * 32 + 2 * e], s1 = s[chunk * 32 + 2 * e + 1];
            float x0, x1, p0, p1;
            unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), c2, n2), x0, x1);
            p0 = ex2_approx(x0);
            p1 = ex2_approx(x1);
            if (e & 1) sum_b = add_f32x2(sum_b, pack_f32x2(p0, p1));
            else sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
            pk[e] = pack_half2(p0, p1);
            if (kWithMax) mx[e & 3] = max3(mx[e & 3], s0, s1);
        }
        if (kStore) {
            tmem_st16(tP + chunk * 16, pk);
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk_out[(chunk - kC0) * 16 + e] = pk[e];
        }
    }
    float lo, hi;
    unpack_f32x2(add_f32x2(sum_a, sum_b), lo, hi);
    return lo + hi;
}

// Read one O row from TMEM, multiply by `f`, write it back.
template <int H>
__device__ __forceinline__ void rescale_o_row(uint32_t tO, float f) {
#pragma unroll
    for (int c0 = 0; c0 < H; c0 += 32) {
        float o[32];
        if constexpr (H % 32 == 0) {
            tmem_ld32(tO + c0, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= f;
            tmem_st32(tO + c0, o);
        } else {  // H == 16
            tmem_ld16(tO + c0, o);
            tmem_wait_ld();
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(o[i] * f);
            tmem_st16(tO + c0, w);
        }
    }
}

// Read one O row from TMEM, multiply by `inv_l`, convert to fp16 and store it with 16-byte stores.
template <int H>
__device__ __forceinline__ void store_o_row(uint32_t tO, float inv_l, __half* dst, bool valid) {
#pragma unroll
    for (int c0 = 0; c0 < H; c0 += 32) {
        float o[32];
        constexpr int n = (H % 32 == 0) ? 32 : 16;
        if constexpr (n == 32) {
            tmem_ld32(tO + c0, o);
        } else {
            tmem_ld16(tO + c0, o);
        }
        tmem_wait_ld();
        if (valid) {
#pragma unroll
            for (int i = 0; i < n; i += 8) {
                uint4 w;
                w.x = pack_half2(o[i] * inv_l, o[i + 1] * inv_l);
                w.y = pack_half2(o[i + 2] * inv_l, o[i + 3] * inv_l);
                w.z = pack_half2(o[i + 4] * inv_l, o[i + 5] * inv_l);
                w.w = pack_half2(o[i + 6] * inv_l, o[i + 7] * inv_l);
                *reinterpret_cast<uint4*>(dst + c0 + i) = w;
            }
        }
    }
}

// Scores of one row (TMEM -> registers).
__device__ __forceinline__ void load_s_row(uint32_t tS, float (&s)[kTile]) {
    tmem_ld32(tS, s);
    tmem_ld32(tS + 32, s + 32);
    tmem_ld32(tS + 64, s + 64);
    tmem_ld32(tS + 96, s + 96);
    tmem_wait_ld();
}

// Columns at or beyond `valid` belong to keys past the end of the sequence.
__device__ __forceinline__ void mask_tail(float (&s)[kTile], int valid) {
#pragma unroll
    for (int i = 0; i < kTile; ++i)
        if (i >= valid) s[i] = -INFINITY;
}

// s[i] += mask[i] * to_score for the first `valid` keys of a tile.  With `vec` (the row starts on a
// 16-byte boundary: L a multiple of 8) whole groups of eight mask values are read with one 16-byte
// load; the ragged remainder and unaligned rows are read value by value.
__device__ __forceinline__ void add_mask_row(float (&s)[kTile], const __half* mrow, int valid, float to_score,
                                             bool vec) {
    if (vec) {
#pragma unroll
        for (int i0 = 0; i0 < kTile; i0 += 8) {
            if (i0 + 8 <= valid) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(mrow + i0));
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ws[e]));
                    s[i0 + 2 * e] = fmaf(f.x, to_score, s[i0 + 2 * e]);
                    s[i0 + 2 * e + 1] = fmaf(f.y, to_score, s[i0 + 2 * e + 1]);
                }
            } else {
#pragma unroll
                for (int i = i0; i < i0 + 8; ++i)
                    if (i < valid) s[i] = fmaf(__half2float(mrow[i]), to_score, s[i]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < kTile; ++i)
            if (i < valid) s[i] = fmaf(__half2float(mrow[i]), to_score, s[i]);
    }
}

// ============================================================================ simple kernel
// grid = ceil(L/128) * R * B CTAs on the x axis (query tile fastest, then head, then batch; one axis
// so that none of the three is held to the 65535 of the y and z axes), block = 128.  Thread t owns
// query row t of the tile (TMEM lane t).
// kPerCtaStatus (only the no-allocation entry point sets it): p.status is an array of one status
// pair per CTA instead of one block per device, so no atomics from different CTAs meet.
template <int H, bool kHasMask, bool kPerCtaStatus = false>
__global__ void __launch_bounds__(128)
fa_fwd_simple(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const Params p) {
    using G = TileGeom<H>;
    constexpr uint32_t kTmemCols = 256;  // S/P in [0,128), O in [128, 128+H)
    enum { BAR_Q = 0, BAR_K, BAR_V, BAR_S, BAR_O, BAR_DRAIN, BAR_COUNT };

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[BAR_COUNT];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5;
    const uint32_t q_tile = blockIdx.x % p.n_q_tiles;
    const uint32_t head = (blockIdx.x / p.n_q_tiles) % p.R, batch = blockIdx.x / (p.n_q_tiles * p.R);
    const int32_t col0 = static_cast<int32_t>(head * H);
    const int32_t q_row0 = static_cast<int32_t>(q_tile * kTile);

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base, sK = sQ + G::kTileBytes, sV = sK + G::kTileBytes;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };
    const WaitCtl ctl{kPerCtaStatus ? p.status + 2u * blockIdx.x : p.status, &abort_flag, kWaitCapCycles,
                      kPerCtaStatus ? nullptr : p.status + 2, p.launch_id};

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < BAR_COUNT; ++i) mbar_init(bar(i), 1);
        abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Everything above touched only this CTA's own state.  From here on global memory is read and
    // written: the kernel before this one in the stream must have completed.
    grid_dep_wait();
    grid_dep_launch();
    if (tid == 96) leave_early_if_launch_failed(ctl);
    const uint32_t tmem_base = tmem_slot;
    const uint32_t lane_off = (warp * 32u) << 16;
    const uint32_t tS = tmem_base + lane_off;          // this thread's score row
    const uint32_t tO = tmem_base + lane_off + 128u;   // this thread's output row
    const uint32_t n_tiles = p.n_kv_tiles;

    // Thread 0 starts every TMA copy and issues every MMA.  Once a wait of this CTA has given up it
    // starts nothing new (`live`), so that at the end at most one copy per barrier is in flight.
    uint32_t nk = 0, nv = 0;   // K and V tiles requested so far (thread 0)
    bool live = true;
    if (tid == 0) {
        load_tile<H>(sQ, &tmQ, bar(BAR_Q), col0, q_row0, batch);
        load_tile<H>(sK, &tmK, bar(BAR_K), col0, 0, batch);
        load_tile<H>(sV, &tmV, bar(BAR_V), col0, 0, batch);
        nk = nv = 1;
    }

    float m = -INFINITY, l = 0.f;
    const uint32_t q_row = q_tile * kTile + tid;
    const bool row_valid = q_row < p.L;

    for (uint32_t j = 0; j < n_tiles; ++j) {
        const uint32_t ph = j & 1u;
        if (tid == 0) {
            if (j == 0) live &= mbar_wait(bar(BAR_Q), 0, ctl, kRoleSimple | BAR_Q);
            live &= mbar_wait(bar(BAR_K), ph, ctl, kRoleSimple | BAR_K);
            tc_fence_after();
            if (live) {
                issue_qk<H>(tmem_base, sQ, sK);
                tc_commit(bar(BAR_S));
            }
        }
        const bool s_ok = mbar_wait(bar(BAR_S), ph, ctl, kRoleSimple | BAR_S);
        tc_fence_after();
        // The K tile is free again: fetch the next one while the softmax runs.
        if (tid == 0 && j + 1 < n_tiles && (live &= s_ok)) {
            load_tile<H>(sK, &tmK, bar(BAR_K), col0, static_cast<int32_t>((j + 1) * kTile), batch);
            ++nk;
        }

        float s[kTile];
        __syncwarp();
        load_s_row(tS, s);
        if constexpr (kHasMask) {
            // additive mask row: mask[batch, q_row, j*128 + i], shared by all heads
            if (row_valid) {
                const __half* mrow = p.mask + (static_cast<size_t>(batch) * p.L + q_row) * p.L +
                                     static_cast<size_t>(j) * kTile;
                const int valid = min(static_cast<int>(p.L - j * kTile), kTile);
                add_mask_row(s, mrow, valid, p.mask_to_score,
                             ((p.L & 7u) | (reinterpret_cast<uintptr_t>(p.mask) & 15u)) == 0u);
            }
        }
        if ((j + 1) * kTile > p.L) mask_tail(s, static_cast<int>(p.L - j * kTile));
        float nmc;
        const float alpha = update_max(m, row_max(s), p.scale_log2, nmc);
        l = l * alpha + exp_and_store_p(s, p.scale_log2, nmc, tS);
        if (j > 0) rescale_o_row<H>(tO, alpha);  // PV(j-1) finished: BAR_O was waited below
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            live &= mbar_wait(bar(BAR_V), ph, ctl, kRoleSimple | BAR_V);
            if (live) {
                issue_pv<H>(tmem_base + 128u, tmem_base, sV, j > 0 ? 1u : 0u);
                tc_commit(bar(BAR_O));
            }
        }
        const bool o_ok = mbar_wait(bar(BAR_O), ph, ctl, kRoleSimple | BAR_O);
        tc_fence_after();
        __syncwarp();
        if (tid == 0 && j + 1 < n_tiles && (live &= o_ok)) {
            load_tile<H>(sV, &tmV, bar(BAR_V), col0, static_cast<int32_t>((j + 1) * kTile), batch);
            ++nv;
        }
    }

    // Y = O / l
    {
        __half* dst = p.y + (static_cast<size_t>(batch) * p.L + q_row) * p.F + head * H;
        store_o_row<H>(tO, 1.f / l, dst, row_valid);
    }
    if (tid == 0 && abort_flag != 0u) {
        // A wait gave up, so the waits behind it returned at once and MMAs this thread issued may
        // still be running.  They retire whatever happened to their inputs; tensor memory and the
        // shared-memory tiles they use are not released before they have.  Likewise the TMA copies
        // this thread started: each of Q, K, V has at most one in flight, the last one requested.
        tc_commit(bar(BAR_DRAIN));
        mbar_wait_certain(bar(BAR_DRAIN), 0, ctl, kRoleDrain | BAR_DRAIN);
        const long long t0 = clock64();
        while (!(mbar_try_wait(bar(BAR_Q), 0) && mbar_try_wait(bar(BAR_K), (nk - 1u) & 1u) &&
                 mbar_try_wait(bar(BAR_V), (nv - 1u) & 1u)) &&
               clock64() - t0 < 200000000LL) {
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ============================================================================ pipelined kernel
template <int H>
struct PipeCfg {
    using G = TileGeom<H>;
    static constexpr int kStages = H == 128 ? 4 : 8;   // ring slots of one K or V tile each
    static constexpr int kQBytes = 2 * G::kTileBytes;  // two query tiles
    static constexpr int kRingBytes = kStages * G::kTileBytes;
    static constexpr int kStageBytes = 4 * 32 * 128;   // epilogue staging: per warp 32 rows x 64 fp16
    static constexpr int kSmemBytes = kQBytes + kRingBytes + kStageBytes + 1024;  // + alignment slack
    static constexpr uint32_t kTmemCols = 512;
    // TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+H) O1 [384,384+H)
    // P (fp16, 64 columns per tile) has columns of its own instead of overwriting its S: the next
    // Q K^T of a tile then does not have to wait for the P V that reads P, only for the softmax warps
    // to have read S, and a tile's softmax passes follow one another without its MMAs in between.
    //   H = 64:   S0 [0,128)  S1 [128,256)  O0 [256,320)  P0 [320,384)  O1 [384,448)  P1 [448,512)
    //   H = 128:  S  [0,128) shared by the two tiles, which use it in turn (scores only live from the
    //             Q K^T until the softmax warps have read them), P0 [128,192)  P1 [192,256)
    //             O0 [256,384)  O1 [384,512)
    static constexpr bool kSharedS = H == 128;
    static constexpr uint32_t kColS0 = 0, kColS1 = kSharedS ? 0 : 128, kColO0 = 256, kColO1 = 384;
    static constexpr uint32_t kColP0 = kSharedS ? 128 : 320, kColP1 = kSharedS ? 192 : 448;
    // Two MMA-issuing warps (one for Q K^T, one for P V) or one for both.  Measured: two win at
    // H = 128 (-3 % SM clocks), one, with its early barriers tested ahead, at H = 64 (-5 %).
    static constexpr bool kTwoIssuers = H == 128;
    // How many 32-key chunks of exponentials a softmax thread takes into registers before it needs
    // the P buffer to be free of the previous step's P V.  Measured at H = 128: 1 (-2.4 %; 2 and 3
    // spill); at H = 64 holding any back costs more than it hides.
    static constexpr int kHeldChunks = H == 128 ? 1 : 0;
};

// Persistent: grid = min(number of SMs, work items), block = 512.  A work item is one pair of
// 128-row query tiles of one (batch, head); CTA c takes items c, c + grid, c + 2*grid, ...  Items
// are numbered query-pair fastest, so the CTAs running at any moment share few heads and their
// K/V tiles stay in L2.  Every role walks the same item list; the key steps of consecutive items
// form one continuous sequence of "global steps", so the two-tile ping-pong never drains: while
// the epilogue warps store item k, the MMA and softmax warps are already in item k+1.
//
// warps 0-3: softmax of query tile 0; 4-7: softmax of tile 1 (each also rescales its O rows in
// the rare steps whose reference maximum moves); 8-11: epilogue (Y = O / l);
// 12: MMA issue (one elected lane) and TMEM owner; 13: TMA producer (one lane); 14: second MMA
// issuing warp at H = 128 (12 issues Q K^T, 14 issues P V); 15: idle.
//
// Per tile and key step: Q K^T -> S; the softmax warps read S into registers and say so (SFREE),
// which lets the next Q K^T into the S buffer; they write P into the tile's P columns once the
// previous step's P V has read them (PV); P V accumulates into O.  Nothing of a tile's next Q K^T
// waits for its P V.
//
// Barrier phases (the parity to wait for is the low bit of the index):
//   per global step g = k*n + j:  S_i (MMA -> softmax), SFREE (softmax -> MMA; at H = 128 one
//                barrier whose phase is the use 2g + i of the shared S buffer), P_i (softmax -> MMA),
//                PV_i (MMA -> softmax and, for the item's last step, epilogue)
//   per item k:  QFULL_i (TMA -> MMA), QEMPTY_i (MMA -> TMA), A_i (softmax -> epilogue),
//                OFREE_i (epilogue -> MMA and softmax)
//   per ring item t (K0 V0 K1 V1 ... across items):  FULL[t % NS], EMPTY[t % NS]
template <int H>
__global__ void __launch_bounds__(512, 1)
fa_fwd_pipelined(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmY,
                 const Params p) {
    using G = TileGeom<H>;
    using C = PipeCfg<H>;
    constexpr int NS = C::kStages;
    enum {
        BAR_QFULL0 = 0, BAR_QFULL1,  // TMA -> MMA: query tile landed
        BAR_QEMPTY0, BAR_QEMPTY1,    // MMA -> TMA: the item's last Q K^T of this tile has retired
        BAR_S0, BAR_S1,              // MMA -> softmax: S tile complete
        BAR_P0, BAR_P1,              // softmax -> MMA: P written (and O rescaled in the rare steps
                                     // that need it); 4 arrivals, one per softmax warp
        BAR_SFREE0, BAR_SFREE1,      // softmax -> MMA: S read into registers (4 arrivals); with the
                                     // one S buffer of H = 128 only the first, one phase per use
        BAR_PV0, BAR_PV1,            // MMA -> softmax (P buffer free, O at rest) and epilogue: P V complete
        BAR_A0, BAR_A1,              // softmax -> epilogue: final row sums in shared memory (4)
        BAR_OFREE0, BAR_OFREE1,      // epilogue -> MMA, softmax: O tile read out (4 arrivals)
        BAR_FINAL,                   // MMA -> itself: every MMA retired
        BAR_FINAL2,                  // the same for the second issuing warp
        BAR_FULL,                    // NS ring barriers TMA -> MMA
        BAR_EMPTY = BAR_FULL + NS,   // NS ring barriers MMA -> TMA
        BAR_COUNT = BAR_EMPTY + NS
    };

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[BAR_COUNT];
    __shared__ float l_buf[2][2][kTile];  // [item parity][tile][row] final row sums
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler
    const uint32_t lane = tid & 31u;
    const uint32_t n = p.n_kv_tiles;
    const uint32_t n_items = p.n_items;
    const uint32_t q_pairs = p.q_pairs;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base;                   // two tiles
    const uint32_t sRing = smem_base + C::kQBytes;   // NS tiles
    const uint32_t sStage = sRing + C::kRingBytes;   // epilogue staging, 4 KiB per epilogue warp
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };
    const WaitCtl ctl{p.status, &abort_flag, kWaitCapCycles, p.status + 2, p.launch_id};

    if (tid == 0) {
        prefetch_tensormap(&tmY);
#pragma unroll
        for (int i = 0; i < BAR_COUNT; ++i) {
            // one arrival per warp (after __syncwarp), not per thread: 128 arrivals on one
            // shared-memory word serialise
            const bool per_warp = (i == BAR_P0 || i == BAR_P1 || i == BAR_SFREE0 || i == BAR_SFREE1 ||
                                   i == BAR_A0 || i == BAR_A1 ||
                                   i == BAR_OFREE0 || i == BAR_OFREE1);
            mbar_init(bar(i), per_warp ? 4u : 1u);
        }
        abort_flag = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
    }
    if (warp == 12) {
        tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Barriers, TMEM and descriptors are set up; nothing of global memory has been touched yet.  In a
    // launch that was allowed to overlap the previous kernel of the stream, wait here for that kernel
    // to complete, then let the next launch's CTAs take the SMs this grid's CTAs leave (they will
    // stop at this same point: the overlap is never deeper than one launch).
    grid_dep_wait();
    grid_dep_launch();
    if (tid == 15 * 32) leave_early_if_launch_failed(ctl);   // warp 15 has no other work
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
#if defined(FA_TRACE) || defined(FA_CYCLES)
    if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[7 * 512] = static_cast<unsigned long long>(clock64());
#endif

    if (warp < 8) {
        // ------------------------------------------------------------------ softmax, tile i
        setmaxnreg_inc<184>();
        const uint32_t i = warp >> 2;
        const uint32_t row = tid & 127u;
        const uint32_t lane_off = ((warp & 3u) * 32u) << 16;
        const uint32_t tS = tmem_base + lane_off + (i ? C::kColS1 : C::kColS0);
        const uint32_t tP = tmem_base + lane_off + (i ? C::kColP1 : C::kColP0);
        const uint32_t tO = tmem_base + lane_off + (i ? C::kColO1 : C::kColO0);
        const float c = p.scale_log2;
        FA_TRACE_DECL
        const bool tr_me = row == 0;
        uint32_t g = 0;   // global step
        uint32_t k = 0;   // item count of this CTA
        for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++k) {
            float m = -INFINITY, l = 0.f;
            for (uint32_t j = 0; j < n; ++j, ++g) {
                mbar_wait(bar(BAR_S0 + i), g & 1u, ctl, kRoleSoftmax | (BAR_S0 + i));
                tc_fence_after();
                __syncwarp();
                if (tr_me) FA_TRACE_EV(1 + i, 1);   // S ready
                float s[kTile];
                const bool ragged = (j + 1) * kTile > p.L;
                const bool first = j == 0;
                load_s_row(tS, s);
                // S is in registers: the MMA warp may overwrite it with the next scores.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(C::kSharedS ? BAR_SFREE0 : BAR_SFREE0 + static_cast<int>(i)));
                // P has one buffer per tile: the previous step's P V must have read it before it is
                // written again.  Where no exponentials are held back in registers the wait is here.
                if constexpr (C::kHeldChunks == 0) {
                    if (g > 0) {
                        mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                        tc_fence_after();
                    }
                }
                if (ragged) mask_tail(s, static_cast<int>(p.L - j * kTile));
                if (first) m = row_max(s);   // first key tile: the reference is its row maximum
                if (tr_me) FA_TRACE_EV(1 + i, 2);   // S in registers
                // Exponentials against the standing reference, with the maximum of the scores taken
                // in the same pass.  The reference only has to move when a score exceeds it by more
                // than 2^8 in the exp2 domain.  P has one buffer per tile and the previous step's P V
                // may still be reading it: the first chunks' exponentials go to registers meanwhile.
                {
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    uint32_t held[16 * (C::kHeldChunks > 0 ? C::kHeldChunks : 1)];
                    float sum = exp_chunks<0, C::kHeldChunks, true, false>(s, c, -m * c, tP, mx4, held);
                    if constexpr (C::kHeldChunks > 0) {
                        if (g > 0) {
                            mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                            tc_fence_after();
                        }
                    }
#pragma unroll
                    for (int ch = 0; ch < C::kHeldChunks; ++ch) tmem_st16(tP + ch * 16, held + ch * 16);
                    sum += exp_chunks<C::kHeldChunks, 4, true>(s, c, -m * c, tP, mx4);
                    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                    const bool moved = (mx - m) * c > kLazyRescaleLog2;
                    if (__any_sync(0xffffffffu, moved)) {
                        // Some row of this warp needs a new reference: redo the warp's exponentials
                        // (rows that keep theirs reproduce the same P) and rescale O by alpha; the
                        // previous step's P V has retired (waited for above), so O is at rest.
                        const float m_new = moved ? mx : m;
                        const float alpha = moved ? ex2_approx((m - m_new) * c) : 1.f;
                        m = m_new;
                        float unused[4];
                        l = l * alpha + exp_chunks<0, 4, false>(s, c, -m * c, tP, unused);
                        // (This wait returns at once.  It is here because with a branch point at this
                        // place of the rare path the compiler allocates the common path without spills.)
                        if (g > 0) mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                        tc_fence_after();
                        __syncwarp();
                        rescale_o_row<H>(tO, alpha);
                    } else {
                        l += sum;
                    }
                }
                if (tr_me) FA_TRACE_EV(1 + i, 5);   // exponentials issued
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_P0 + i));
                if (tr_me) FA_TRACE_EV(1 + i, 4);   // P signalled
            }
            // Hand the row sums to the epilogue.  The A barrier may run at most one phase ahead of
            // the epilogue's wait, so the previous item's O must have been read out first (always
            // true already when an item has two or more key steps).
            if (k > 0) mbar_wait(bar(BAR_OFREE0 + i), (k - 1u) & 1u, ctl, kRoleSoftmax | (BAR_OFREE0 + i));
            l_buf[k & 1u][i][row] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAR_A0 + i));
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ epilogue: Y = O / l
        // Each warp owns 32 rows of the tile.  It reads them from TMEM 64 columns at a time, scales
        // by 1/l, rounds to fp16 and writes 16-byte vectors into its 4 KiB staging buffer (rows of
        // 128 bytes, 128-byte swizzle), which one TMA store sends to Y: the warp is not held up by
        // scattered global stores and the O tile is handed back as soon as it is in registers.
        setmaxnreg_dec<64>();
        const uint32_t row = tid & 127u;
        const uint32_t wq = warp & 3u;
        const uint32_t lane_off = (wq * 32u) << 16;
        const uint32_t stage = sStage + wq * 4096u;
        uint32_t k = 0;
        for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++k) {
            const uint32_t q_pair = item % q_pairs, bh = item / q_pairs;
            const uint32_t head = bh % p.R, batch = bh / p.R;
#pragma unroll
            for (uint32_t i = 0; i < 2; ++i) {
                // this wait lasts for a whole item: poll every 100 ns
                mbar_wait_relaxed(bar(BAR_A0 + i), k & 1u, ctl, kRoleEpilogue | (BAR_A0 + i), 100);
                const float inv_l = 1.f / l_buf[k & 1u][i][row];
                // The item's last P V of this tile.  Every earlier phase of this barrier has
                // completed by the time the softmax warps signalled and the next phase needs this
                // epilogue's OFREE arrival, so the parity test is unambiguous.
                mbar_wait(bar(BAR_PV0 + i), (k * n + n - 1u) & 1u, ctl, kRoleEpilogue | (BAR_PV0 + i));
                tc_fence_after();
                __syncwarp();
                const uint32_t tO = tmem_base + lane_off + (i ? C::kColO1 : C::kColO0);
                const int32_t row0 = static_cast<int32_t>((q_pair * 2u + i) * kTile + wq * 32u);
#pragma unroll
                for (int half = 0; half < H / 64; ++half) {
                    // the previous store out of this staging buffer must have read it completely
                    if (lane == 0) bulk_wait_read_all();
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {   // 16 columns at a time keeps this role within 64 registers
                        float o[16];
                        tmem_ld16(tO + half * 64 + c * 16, o);
                        tmem_wait_ld();
                        if (half == H / 64 - 1 && c == 3) {
                            // the whole O tile has left TMEM: the MMA warp may overwrite it
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar(BAR_OFREE0 + i));
                        }
#pragma unroll
                        for (int v4 = 0; v4 < 2; ++v4) {
                            const uint32_t w0 = pack_half2(o[v4 * 8 + 0] * inv_l, o[v4 * 8 + 1] * inv_l);
                            const uint32_t w1 = pack_half2(o[v4 * 8 + 2] * inv_l, o[v4 * 8 + 3] * inv_l);
                            const uint32_t w2 = pack_half2(o[v4 * 8 + 4] * inv_l, o[v4 * 8 + 5] * inv_l);
                            const uint32_t w3 = pack_half2(o[v4 * 8 + 6] * inv_l, o[v4 * 8 + 7] * inv_l);
                            // logical 16-byte chunk c*2+v4 of row `lane`, 128-byte swizzle
                            const uint32_t chunk = static_cast<uint32_t>(c * 2 + v4) ^ (lane & 7u);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128u + chunk * 16u),
                                         "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                                         : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < static_cast<int32_t>(p.L)) {   // rows past L are clipped by the store
                        tma_store_3d(&tmY, stage, static_cast<int32_t>(head * H + half * 64), row0,
                                     static_cast<int32_t>(batch));
                        bulk_commit_group();
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();   // Y is complete before the CTA leaves
    } else {
        setmaxnreg_dec<80>();
        if (warp == 12 || (C::kTwoIssuers && warp == 14)) {
            // -------------------------------------------------------------- MMA issue
            // The whole warp walks the loop (uniform control flow keeps descriptors in uniform
            // registers); one elected lane issues the MMAs and commits.  With P in columns of its
            // own, warp 12 issues the Q K^T of both tiles and warp 14 their P V: the two streams
            // depend on nothing of one another (different TMEM columns, different ring slots), and
            // a barrier wait of one issuing thread, which costs it 150-300 clocks during which it
            // issues nothing, is then covered by the MMAs the other warp has queued.
            const bool leader = elect_one();
            const uint32_t tS0 = tmem_base + C::kColS0, tS1 = tmem_base + C::kColS1;
            const uint32_t tO0 = tmem_base + C::kColO0, tO1 = tmem_base + C::kColO1;
            const uint32_t tP0 = tmem_base + C::kColP0, tP1 = tmem_base + C::kColP1;
            auto slot_addr = [&](uint32_t t) { return sRing + (t % NS) * G::kTileBytes; };
            // Once one of this warp's waits has given up (`ok` false) it issues nothing more: what it
            // would multiply has not arrived.
            bool ok = true;
            auto mwait = [&](uint32_t b, uint32_t parity, const WaitCtl& wc, uint32_t code) {
                ok &= mbar_wait(b, parity, wc, code);
            };
            auto wait_full = [&](uint32_t t) {
                mwait(bar(BAR_FULL + (t % NS)), (t / NS) & 1u, ctl, kRoleMma | (BAR_FULL + (t % NS)));
            };
            auto free_slot = [&](uint32_t t) { tc_commit(bar(BAR_EMPTY + (t % NS))); };
#ifdef FA_TRACE
            uint32_t tr_n = 0;
            const bool tr_on = leader && p.trace != nullptr && blockIdx.x == p.trace_cta;
#endif
            const uint32_t my_items = blockIdx.x < n_items ? (n_items - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
            const uint32_t steps = my_items * n;   // global steps of this CTA
            // ring item 2g is the K tile of global step g, item 2g+1 its V tile
            if (steps > 0 && warp == 12) {
                // S tiles of the very first step
                mwait(bar(BAR_QFULL0), 0, ctl, kRoleMma | BAR_QFULL0);
                wait_full(0);
                tc_fence_after();
                if (leader && ok) {
                    issue_qk<H>(tS0, sQ, slot_addr(0));
                    tc_commit(bar(BAR_S0));
                    if (n == 1) tc_commit(bar(BAR_QEMPTY0));
                }
                mwait(bar(BAR_QFULL1), 0, ctl, kRoleMma | BAR_QFULL1);
                // one S buffer for both tiles: tile 0's scores must have been read first
                if constexpr (C::kSharedS) mwait(bar(BAR_SFREE0), 0, ctl, kRoleMma | BAR_SFREE0);
                tc_fence_after();
                if (leader && ok) {
                    issue_qk<H>(tS1, sQ + G::kTileBytes, slot_addr(0));
                    tc_commit(bar(BAR_S1));
                    if (n == 1) tc_commit(bar(BAR_QEMPTY1));
                    free_slot(0);
                }
            }
            uint32_t k = 0, j = 0;   // item and key step of global step g
            if constexpr (C::kTwoIssuers) {
                mbar_poll_declare();
                bool polled = false;
                if (warp == 12) {
                    // Q K^T stream: for every step g the scores of step g + 1, tile 0 then tile 1, each
                    // as soon as the softmax warps have read what the S buffer holds.  That K has
                    // landed is known long before; it is tested ahead of the previous step's last
                    // MMAs and the answer read after them (mbar_poll_begin).
                    for (uint32_t g = 0; g + 1 < steps; ++g) {
                        const uint32_t tk = 2 * g + 2;
                        const bool next_new_item = j + 1 == n;    // step g + 1 opens item k + 1
                        if (!(polled && mbar_poll_end<0>())) wait_full(tk);
                        if (next_new_item) mwait(bar(BAR_QFULL0), (k + 1u) & 1u, ctl, kRoleMma | BAR_QFULL0);
                        // With one S buffer its uses are numbered 2g + i (tile i, step g) and use u
                        // needs the reading of use u - 1 (one barrier, phase = use); with one buffer
                        // per tile the reading of step g of that tile.
                        if constexpr (C::kSharedS) mwait(bar(BAR_SFREE0), 1u, ctl, kRoleMma | BAR_SFREE0);
                        else mwait(bar(BAR_SFREE0), g & 1u, ctl, kRoleMma | BAR_SFREE0);
                        FA_TRACE_EV(0, 11);  // S0 read by the softmax warps
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS0, sQ, slot_addr(tk));
                            tc_commit(bar(BAR_S0));
                            // the Q K^T of an item's last key step is its last use of the query tile
                            if (next_new_item ? n == 1 : j + 2 == n) tc_commit(bar(BAR_QEMPTY0));
                        }
                        FA_TRACE_EV(0, 4);   // next Q K^T of tile 0 issued
                        if (next_new_item) mwait(bar(BAR_QFULL1), (k + 1u) & 1u, ctl, kRoleMma | BAR_QFULL1);
                        if constexpr (C::kSharedS) mwait(bar(BAR_SFREE0), 0u, ctl, kRoleMma | BAR_SFREE0);
                        else mwait(bar(BAR_SFREE1), g & 1u, ctl, kRoleMma | BAR_SFREE1);
                        FA_TRACE_EV(0, 12);  // S1 read by the softmax warps
                        tc_fence_after();
                        polled = g + 2 < steps;
                        if (polled) {
                            const uint32_t nk = tk + 2;
                            mbar_poll_begin<0>(bar(BAR_FULL + (nk % NS)), (nk / NS) & 1u);
                        }
                        if (leader && ok) {
                            issue_qk<H>(tS1, sQ + G::kTileBytes, slot_addr(tk));
                            tc_commit(bar(BAR_S1));
                            if (next_new_item ? n == 1 : j + 2 == n) tc_commit(bar(BAR_QEMPTY1));
                            free_slot(tk);
                        }
                        FA_TRACE_EV(0, 7);   // next Q K^T of tile 1 issued
                        if (++j == n) { j = 0; ++k; }
                    }
                } else {
                    // P V stream: for every step the products of tile 0 and tile 1 as their P arrive.
                    for (uint32_t g = 0; g < steps; ++g) {
                        const uint32_t tv = 2 * g + 1;
                        const uint32_t acc = j > 0 ? 1u : 0u;
                        if (!(polled && mbar_poll_end<1>())) wait_full(tv);
                        if (j == 0 && k > 0) mwait(bar(BAR_OFREE0), (k - 1u) & 1u, ctl, kRoleMma | BAR_OFREE0);
                        mwait(bar(BAR_P0), g & 1u, ctl, kRoleMma | BAR_P0);
                        FA_TRACE_EV(3, 2);   // P0 ready
                        tc_fence_after();
                        if (leader && ok) {
                            issue_pv<H>(tO0, tP0, slot_addr(tv), acc);
                            tc_commit(bar(BAR_PV0));
                        }
                        FA_TRACE_EV(3, 8);   // P V of tile 0 issued
                        if (j == 0 && k > 0) mwait(bar(BAR_OFREE1), (k - 1u) & 1u, ctl, kRoleMma | BAR_OFREE1);
                        mwait(bar(BAR_P1), g & 1u, ctl, kRoleMma | BAR_P1);
                        FA_TRACE_EV(3, 5);   // P1 ready
                        tc_fence_after();
                        polled = g + 1 < steps;
                        if (polled) {
                            const uint32_t nv = tv + 2;
                            mbar_poll_begin<1>(bar(BAR_FULL + (nv % NS)), (nv / NS) & 1u);
                        }
                        if (leader && ok) {
                            issue_pv<H>(tO1, tP1, slot_addr(tv), acc);
                            tc_commit(bar(BAR_PV1));
                            free_slot(tv);
                        }
                        FA_TRACE_EV(3, 10);  // P V of tile 1 issued
                        if (++j == n) { j = 0; ++k; }
                    }
                }
            } else {
                // P in columns of its own: per tile, the next step's Q K^T goes out as soon as the
                // softmax warps have read S, ahead of the P V of this step.  The tiles that have landed
                // and the S that has been read are known long before the MMA warp needs to know, so
                // those barriers are tested ahead of a group of MMAs and the answer is read after it
                // (mbar_poll_begin); only the waits for P block.
                mbar_poll_declare();
                bool polled = false;   // predicates 0-2 hold answers for this step
                for (uint32_t g = 0; g < steps; ++g) {
                    const uint32_t tv = 2 * g + 1, tk = 2 * g + 2;
                    const bool more = g + 1 < steps;          // a next global step exists
                    const bool next_new_item = j + 1 == n;    // ... and it opens item k + 1
                    const uint32_t acc = j > 0 ? 1u : 0u;
                    {
                        uint32_t ok_v = 0, ok_k = 0, ok_s0 = 0;
                        if (polled) {
                            ok_v = mbar_poll_end<0>();
                            ok_k = mbar_poll_end<1>();
                            ok_s0 = mbar_poll_end<2>();
                        }
                        if (!ok_v) wait_full(tv);
                        if (more) {
                            if (!ok_k) wait_full(tk);
                            if (next_new_item) mwait(bar(BAR_QFULL0), (k + 1u) & 1u, ctl, kRoleMma | BAR_QFULL0);
                            if (!ok_s0) mwait(bar(BAR_SFREE0), g & 1u, ctl, kRoleMma | BAR_SFREE0);
                        }
                    }
                    if (j == 0 && k > 0) mwait(bar(BAR_OFREE0), (k - 1u) & 1u, ctl, kRoleMma | BAR_OFREE0);
                    FA_TRACE_EV(0, 1);   // V and next K landed, S0 read by the softmax warps
                    // tile 0
                    if (more) {
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS0, sQ, slot_addr(tk));
                            tc_commit(bar(BAR_S0));
                            // the Q K^T of an item's last key step is its last use of the query tile
                            if (next_new_item ? n == 1 : j + 2 == n) tc_commit(bar(BAR_QEMPTY0));
                        }
                    }
                    FA_TRACE_EV(0, 4);   // next Q K^T of tile 0 issued
                    mwait(bar(BAR_P0), g & 1u, ctl, kRoleMma | BAR_P0);
                    FA_TRACE_EV(0, 2);   // P0 ready
                    tc_fence_after();
                    if (more) mbar_poll_begin<3>(bar(BAR_SFREE1), g & 1u);   // read behind the P V below
                    if (leader && ok) {
                        issue_pv<H>(tO0, tP0, slot_addr(tv), acc);
                        tc_commit(bar(BAR_PV0));
                    }
                    FA_TRACE_EV(0, 8);   // P V of tile 0 issued
                    // tile 1
                    if (more && next_new_item) mwait(bar(BAR_QFULL1), (k + 1u) & 1u, ctl, kRoleMma | BAR_QFULL1);
                    if (j == 0 && k > 0) mwait(bar(BAR_OFREE1), (k - 1u) & 1u, ctl, kRoleMma | BAR_OFREE1);
                    if (more) {
                        if (!mbar_poll_end<3>()) mwait(bar(BAR_SFREE1), g & 1u, ctl, kRoleMma | BAR_SFREE1);
                        FA_TRACE_EV(0, 12);  // S1 read by the softmax warps
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS1, sQ + G::kTileBytes, slot_addr(tk));
                            tc_commit(bar(BAR_S1));
                            if (next_new_item ? n == 1 : j + 2 == n) tc_commit(bar(BAR_QEMPTY1));
                            free_slot(tk);
                        }
                    }
                    FA_TRACE_EV(0, 7);   // next Q K^T of tile 1 issued
                    mwait(bar(BAR_P1), g & 1u, ctl, kRoleMma | BAR_P1);
                    FA_TRACE_EV(0, 5);   // P1 ready
                    tc_fence_after();
                    // what the next step starts with: test now, read at the top of the next step
                    polled = more;
                    if (more) {
                        const uint32_t nv = tv + 2, nk = tk + 2;
                        mbar_poll_begin<0>(bar(BAR_FULL + (nv % NS)), (nv / NS) & 1u);
                        mbar_poll_begin<1>(bar(BAR_FULL + (nk % NS)), (nk / NS) & 1u);
                        mbar_poll_begin<2>(bar(BAR_SFREE0), (g + 1u) & 1u);
                    }
                    if (leader && ok) {
                        issue_pv<H>(tO1, tP1, slot_addr(tv), acc);
                        tc_commit(bar(BAR_PV1));
                        free_slot(tv);
                    }
                    FA_TRACE_EV(0, 10);  // P V of tile 1 issued
                    if (++j == n) { j = 0; ++k; }
                }
            }
            const int bar_final = warp == 12 ? BAR_FINAL : BAR_FINAL2;
            // Every MMA this warp issued has to retire before the CTA releases tensor memory and shared
            // memory, whether or not a wait gave up on the way: this wait does not look at the abort flag.
            if (leader) tc_commit(bar(bar_final));
            __syncwarp();
            mbar_wait_certain(bar(bar_final), 0, ctl, kRoleMma | static_cast<uint32_t>(bar_final));
        } else if (warp == 13 && elect_one()) {
            // -------------------------------------------------------------- TMA producer
            uint32_t t = 0;           // ring item
            uint32_t k = 0;           // item count of this CTA
            bool stop = false;
            bool q_pending[2] = {false, false};
            for (uint32_t item = blockIdx.x; item < n_items && !stop; item += gridDim.x, ++k) {
                const uint32_t q_pair = item % q_pairs, bh = item / q_pairs;
                const int32_t col0 = static_cast<int32_t>((bh % p.R) * H);
                const int32_t batch = static_cast<int32_t>(bh / p.R);
                const int32_t q_row0 = static_cast<int32_t>(q_pair * 2u * kTile);
                for (uint32_t tt = 0; tt < 2 * n; ++tt, ++t) {
                    if (tt < 2) {
                        // query tile tt of this item, once the previous item has let go of the buffer
                        if (k > 0 && !mbar_wait(bar(BAR_QEMPTY0 + tt), (k - 1u) & 1u, ctl,
                                                kRoleProducer | (BAR_QEMPTY0 + tt))) { stop = true; break; }
                        load_tile<H>(sQ + tt * G::kTileBytes, &tmQ, bar(BAR_QFULL0 + tt), col0,
                                     q_row0 + static_cast<int32_t>(tt * kTile), batch);
                        q_pending[tt] = true;
                    }
                    const uint32_t slot = t % NS;
                    if (!mbar_wait(bar(BAR_EMPTY + slot), ((t / NS) & 1u) ^ 1u, ctl,
                                   kRoleProducer | (BAR_EMPTY + slot))) { stop = true; break; }
                    load_tile<H>(sRing + slot * G::kTileBytes, (tt & 1u) ? &tmV : &tmK, bar(BAR_FULL + slot),
                                 col0, static_cast<int32_t>((tt >> 1) * kTile), batch);
                }
            }
            if (abort_flag != 0u) {
                // Do not leave the CTA while one of its own copies may still be landing.
                const uint32_t first = t > NS ? t - NS : 0u;
                for (uint32_t u = first; u < t; ++u) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar(BAR_FULL + (u % NS)), (u / NS) & 1u) &&
                           clock64() - t0 < 200000000LL) {
                    }
                }
                for (uint32_t tt = 0; tt < 2; ++tt) {
                    const long long t0 = clock64();
                    while (q_pending[tt] && !mbar_try_wait(bar(BAR_QFULL0 + tt), (k > 0 ? k - 1u : 0u) & 1u) &&
                           clock64() - t0 < 200000000LL) {
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
#if defined(FA_TRACE) || defined(FA_CYCLES)
    if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[7 * 512 + 1] = static_cast<unsigned long long>(clock64());
#endif
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Self-test of the bounded wait: one warp waits on an mbarrier that nothing ever completes, with a
// short cap.  The wait must give up, record `code` in the status word and return normally.
__global__ void fa_selftest_bounded_wait(uint32_t* status, uint32_t code, long long cap_cycles,
                                         uint32_t* returned) {
    __shared__ __align__(8) uint64_t bar_mem;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar_mem), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const WaitCtl ctl{status, &abort_flag, cap_cycles};
    const bool ok = mbar_wait(smem_u32(&bar_mem), 0, ctl, code);
    __syncthreads();
    if (threadIdx.x == 0) *returned = ok ? 1u : 2u;  // 2 = gave up, as it must
}

}  // namespace fa
