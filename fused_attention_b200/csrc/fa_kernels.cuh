// Fused multi-head attention forward for sm_100a:  Y = softmax(Q K^T / sqrt(H)) V.
//
// Two kernels share the same arithmetic:
//   fa_fwd_simple<H, kHasMask>  one 128-row query tile per CTA, 128 threads, every step in program
//                               order.  Covers every head_dim (16, 32, 64, 128), the additive mask
//                               and tiny problems; several CTAs per SM overlap one another.
//   fa_fwd_pipelined<H, kHasMask>  two 128-row query tiles per CTA, 512 threads split into roles
//                               (2 softmax warpgroups, 1 epilogue warpgroup, 1 or 2 MMA warps, 1 TMA
//                               warp, 1 warp for the mask tiles); K/V stream through a shared-memory
//                               ring; the softmax of one tile overlaps the MMAs of the other.
//                               H in {64, 128}.
// fa_pair.cuh holds a third, fa_fwd_pair<kHasMask>: the same roles on pairs of CTAs at H = 128.
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
    uint32_t mask_tma;    // pipelined kernel with a mask: 1 = mask tiles come through TMA (rows 16-byte aligned)
    // schedule of the pipelined kernel (see Plan) and the scratch of a divided tail round
    uint32_t full_rounds;  // rounds of whole items: item = cta + k * grid
    uint32_t tail_items;   // items after the full rounds whose key steps are divided among the CTAs
    uint32_t tail_steps;   // tail_items * n_kv_tiles, or 0 when nothing is divided
    uint32_t tail_grid;    // the first tail_grid CTAs share the tail key steps (at most the grid)
    float4* part_o;        // [2 * grid slots][2 tiles][H/4][128 rows] numerators of partial segments, fp32
    float2* part_ml;       // [2 * grid slots][2 tiles][128 rows] {reference maximum, row sum}
    uint32_t* part_cnt;    // [tail item][2 tiles][4 warps] parts counted in; zero between launches
    uint32_t part_slots;   // scratch slots behind part_o / part_ml (two per CTA of the largest grid)
#ifdef FA_CYCLES
    unsigned long long* cycles;  // 64 records (launch_id % 64) of CTA 0: {globaltimer at entry, globaltimer after the
                                 // wait for the previous kernel, globaltimer at the end, clock64 from that wait to the end}
#endif
};

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

#ifdef FA_DEBUG
// Checked build: fill in the CTA's check context (one thread) and poison its tile area with NaN (all threads).
// The caller synchronises the CTA afterwards, before the first copy is started.
__device__ __forceinline__ void dbg_begin(const Params& p, const WaitCtl& ctl, uint32_t smem_base, uint32_t bytes) {
    if (threadIdx.x == 0) {
        g_dbg.smem_lo = smem_base;
        g_dbg.smem_hi = smem_base + bytes;
        g_dbg.F = p.F;
        g_dbg.L = p.L;
        g_dbg.B = p.B;
        g_dbg.tmem_base = 0;
        g_dbg.tmem_cols = 512;
        g_dbg.ctl = ctl;
    }
    for (uint32_t off = threadIdx.x * 16u; off < bytes; off += blockDim.x * 16u)
        st_shared_v4(smem_base + off, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    fence_proxy_async_smem();
}
// ... and, once tensor memory has been allocated, its extent (one thread; the caller synchronises).
__device__ __forceinline__ void dbg_tmem(uint32_t base, uint32_t cols) {
    g_dbg.tmem_base = base;
    g_dbg.tmem_cols = cols;
}
#endif

// Ask for one tile (all its boxes) to be brought into L2.
template <int H>
__device__ __forceinline__ void prefetch_tile_l2(const CUtensorMap* map, int32_t col0, int32_t row0, int32_t batch) {
    using G = TileGeom<H>;
#pragma unroll
    for (int b = 0; b < G::kBoxes; ++b) tma_prefetch_l2_3d(map, col0 + b * G::kBoxCols, row0, batch);
}

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
// A row sum of P below this proves that no P of the row exceeds 2^kLazyRescaleLog2 (the margin of one covers
// the error of ex2.approx at the threshold).
constexpr float kLazyRescaleSum = 255.f;
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

// One O row from TMEM, multiplied by `inv_l` and converted to fp16, into a staging area in shared memory from
// where TMA stores it: for a thread with registers to spare (a softmax thread), the whole row in one round trip.
// The area holds, per 64 columns, one box of the Y map (32 rows of 128 bytes with the 128-byte swizzle: 16-byte
// piece c of row r at piece c ^ (r & 7)); `stage` is 1024-byte aligned, `lane` the row within the box.
template <int H>
__device__ __forceinline__ void stage_o_row(uint32_t tO, float inv_l, uint32_t stage, uint32_t lane) {
    static_assert(H % 64 == 0, "boxes of 64 columns");
    float o[H];
#pragma unroll
    for (int c0 = 0; c0 < H; c0 += 32) tmem_ld32(tO + c0, o + c0);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < H; i += 8) {
        const uint32_t w0 = pack_half2(o[i] * inv_l, o[i + 1] * inv_l);
        const uint32_t w1 = pack_half2(o[i + 2] * inv_l, o[i + 3] * inv_l);
        const uint32_t w2 = pack_half2(o[i + 4] * inv_l, o[i + 5] * inv_l);
        const uint32_t w3 = pack_half2(o[i + 6] * inv_l, o[i + 7] * inv_l);
        const uint32_t piece = static_cast<uint32_t>((i % 64) / 8) ^ (lane & 7u);
        st_shared_v4(stage + static_cast<uint32_t>(i / 64) * 4096u + lane * 128u + piece * 16u, w0, w1, w2, w3);
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

// s[i] += mask[i] * to_score for the first `valid` keys of a tile.  Every thread reads its own row of the
// mask, so the lanes of a warp touch 32 different lines per load instruction whatever its width: the wider the
// load, the fewer passes through the load unit.  `align` is the alignment in bytes that every row start of
// this call is known to have (32, 16 or 2): whole groups of 16 (8) mask values are read with one 32-byte
// (16-byte) load; the ragged remainder and unaligned rows are read value by value.
__device__ __forceinline__ void add_mask_row(float (&s)[kTile], const __half* mrow, int valid, float to_score,
                                             uint32_t align) {
    if (align >= 32u) {
#pragma unroll
        for (int i0 = 0; i0 < kTile; i0 += 16) {
            if (i0 + 16 <= valid) {
                uint32_t w[8];
                ldg_256(mrow + i0, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                    s[i0 + 2 * e] = fmaf(f.x, to_score, s[i0 + 2 * e]);
                    s[i0 + 2 * e + 1] = fmaf(f.y, to_score, s[i0 + 2 * e + 1]);
                }
            } else {
#pragma unroll
                for (int i = i0; i < i0 + 16; ++i)
                    if (i < valid) s[i] = fmaf(__half2float(mrow[i]), to_score, s[i]);
            }
        }
    } else if (align >= 16u) {
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

// The same from a mask tile that TMA has brought into shared memory: two boxes of 128 rows x 64 keys, rows of
// 128 bytes with the 128-byte swizzle (16-byte chunk c of row r lies at chunk c ^ (r & 7)).  Keys and rows
// beyond the end of the sequence were filled with zeros.
__device__ __forceinline__ void add_mask_tile_row(float (&s)[kTile], uint32_t smask, uint32_t row, float to_score) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
            ld_shared_v4(smask + b * (kTile * 128) + row * 128u + ((static_cast<uint32_t>(c) ^ (row & 7u)) * 16u), w);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                const int i = b * 64 + c * 8 + 2 * e;
                // one packed multiply-add for the two scores (the same two roundings as two scalar ones)
                unpack_f32x2(fma_f32x2(pack_f32x2(f.x, f.y), pack_f32x2(to_score, to_score), pack_f32x2(s[i], s[i + 1])),
                             s[i], s[i + 1]);
            }
        }
    }
}

// What every mask row start of a call is aligned to: rows are L fp16 values apart from the base address.
__device__ __forceinline__ uint32_t mask_row_alignment(const Params& p) {
    const uint32_t bits = (p.L * 2u) | static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.mask));
    return (bits & 31u) == 0u ? 32u : ((bits & 15u) == 0u ? 16u : 2u);
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
#ifdef FA_DEBUG
    dbg_begin(p, ctl, smem_base, 3u * G::kTileBytes);
#endif
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
#ifdef FA_DEBUG
    if (tid == 0) dbg_tmem(tmem_slot, kTmemCols);
    __syncthreads();
#endif
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
                add_mask_row(s, mrow, valid, p.mask_to_score, mask_row_alignment(p));
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

// Time line of the key-step loop, only in builds with -DFA_CYCLES -DFA_TIMELINE (the pair kernel has the stamps):
// lane 0 of one warp per role of CTA 0 writes its SM clock at event `ev` of global key step `g` into word
// 256 + ((role * 256 + g) * 8 + ev) of the buffer given to fa_b200_debug_cycles (9 * 1024 words in such a build);
// steps beyond 255 are not recorded.  Roles: 0, 1 a softmax warp of query tile 0, 1; 2 the warp issuing Q K^T;
// 3 the warp issuing P V.  Events are listed where the stamps are.
#if defined(FA_CYCLES) && defined(FA_TIMELINE)
#define FA_STAMP(role, g, ev)                                                                         \
    do {                                                                                              \
        if (p.cycles != nullptr && blockIdx.x == 0 && lane == 0 && (g) < 256u)                        \
            p.cycles[256u + (((role) * 256u + (g)) * 8u) + (ev)] = static_cast<unsigned long long>(clock64()); \
    } while (0)
#else
#define FA_STAMP(role, g, ev) do { } while (0)
#endif

// ============================================================================ pipelined kernel
template <int H, bool kHasMask = false>
struct PipeCfg {
    using G = TileGeom<H>;
    // ring slots of one K or V tile each; with a mask a quarter of the ring makes room for one mask tile
    static constexpr int kStages = (H == 128 ? 4 : 8) * (kHasMask ? 3 : 4) / 4;
    // Buffers for the two query tiles of a segment.  With two of them (H = 64, where they fit) the next segment's
    // query tiles, and behind them its K and V tiles, are on their way while this segment still multiplies: the
    // producer no longer stops at every segment boundary until the last Q K^T has let go of the one buffer.
    // Measured: 1 to 1.5 % fewer SM clocks per CTA on shapes of two to sixteen key steps per segment.
    static constexpr int kQBufs = H == 64 ? 2 : 1;
    static constexpr int kQBytes = 2 * G::kTileBytes;  // two query tiles
    static constexpr int kRingBytes = kStages * G::kTileBytes;
    static constexpr int kMaskBytes = kHasMask ? kTile * kTile * 2 : 0;   // one 128 x 128 fp16 mask tile (two boxes of 64 keys)
    static constexpr int kStageBytes = 4 * 32 * 128;   // epilogue staging: per warp 32 rows x 64 fp16
    static constexpr int kSmemBytes = kQBufs * kQBytes + kRingBytes + kMaskBytes + kStageBytes + 1024;  // + alignment slack
    static constexpr uint32_t kTmemCols = 512;
    // TMEM columns.  P (fp16, 64 columns per tile) has columns of its own instead of overwriting its
    // S: the next Q K^T of a tile then does not have to wait for the P V that reads P, only for the
    // softmax warps to have read S, and a tile's softmax passes follow one another without its MMAs
    // in between.
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
    // Whether the softmax warps write Y of the CTA's last segment themselves when it is a whole work item (both
    // tiles at once, nothing being left to overlap an epilogue with) instead of handing it to the epilogue warps.
    // Measured: H = 128 1 to 2 % fewer SM clocks on launches of one or two items per CTA, nothing on long ones;
    // H = 64 2 % more on every shape (the extra code costs the row pass registers).
    static constexpr bool kSoftmaxWritesLast = H == 128;
};

// Into how many parts the key axis of one work item may be divided (see Plan).
constexpr uint32_t kMaxParts = 3;

// What one CTA of the pipelined kernel does: a list of SEGMENTS, each a run of consecutive key steps
// of one work item (a pair of 128-row query tiles of one (batch, head)).
//   - `whole` segments are whole items (all n key steps), taken round-robin: item = cta + k * grid.
//     Items are numbered query-pair fastest, so the CTAs running at any moment share few heads and
//     their K/V tiles stay in L2.  They come before the CTA's tail segments (below).
//   - When the items do not fill a whole number of rounds, the launcher may divide the last, partial
//     round (Params::tail_items items after full_rounds * grid, T = tail_steps = tail_items * n key
//     steps in all) evenly among the first tg = Params::tail_grid CTAs: CTA c < tg takes the tail key
//     steps [c*T/tg, (c+1)*T/tg), numbered item by item.  That range is never longer than n, so it
//     touches at most two items: up to two tail segments, the first ending an item (or lying inside
//     one), the second starting the next item at step 0; and never shorter than n/2, so no item is
//     cut into more than three parts.
// A segment that does not cover all n key steps is PARTIAL: its epilogue does not write Y but adds
// its (reference maximum, row sum, numerator) to the item's other parts, see the epilogue role.
struct Plan {
    uint32_t whole;     // whole-item segments of this CTA: segments 0 .. whole-1
    uint32_t ntail;     // tail segments of this CTA (0, 1 or 2): segments whole .. nseg-1
    uint32_t nseg;      // all segments of this CTA
    uint32_t steps;     // all key steps of this CTA
    uint32_t t_item0;   // first tail segment: index of its item among the tail items,
    uint32_t t_j00;     //   its first key step,
    uint32_t t_len0;    //   its length (0 = no tail segment)
    uint32_t t_len1;    // second tail segment: item t_item0 + 1 from key step 0, this long (0 = none)
};

__device__ __forceinline__ Plan make_plan(const Params& p) {
    Plan pl;
    const uint32_t n = p.n_kv_tiles, grid = gridDim.x, c = blockIdx.x;
    pl.t_item0 = pl.t_j00 = pl.t_len0 = pl.t_len1 = 0;
    if (p.tail_steps == 0) {
        pl.whole = c < p.n_items ? (p.n_items - c + grid - 1u) / grid : 0u;
    } else {
        pl.whole = p.full_rounds;
        const uint32_t tg = p.tail_grid;                       // the launcher keeps tail_steps * tail_grid below 2^32
        const uint32_t a = c < tg ? c * p.tail_steps / tg : 0u;
        const uint32_t b = c < tg ? (c + 1u) * p.tail_steps / tg : 0u;
        if (b > a) {
            pl.t_item0 = a / n;
            pl.t_j00 = a - pl.t_item0 * n;
            pl.t_len0 = min(n - pl.t_j00, b - a);
            pl.t_len1 = (b - a) - pl.t_len0;
        }
    }
    pl.ntail = (pl.t_len0 ? 1u : 0u) + (pl.t_len1 ? 1u : 0u);
    pl.nseg = pl.whole + pl.ntail;
    pl.steps = pl.whole * n + pl.t_len0 + pl.t_len1;
    return pl;
}

struct Seg {
    uint32_t item;       // work item: q_pair = item % q_pairs, (batch, head) = item / q_pairs
    uint32_t j0, len;    // key steps [j0, j0 + len)
    bool partial;        // fewer than all n key steps
};
// Of a tail segment k (k >= t0 = number of whole segments): index of its item among the tail items; this
// CTA's scratch slot for the part (two per CTA).  Looked up where they are needed rather than kept in
// registers.
template <typename PlanRef>
__device__ __forceinline__ uint32_t seg_tail_item(PlanRef& pl, uint32_t t0, uint32_t k) { return pl.t_item0 + (k - t0); }
__device__ __forceinline__ uint32_t seg_slot(uint32_t t0, uint32_t k) { return 2u * blockIdx.x + (k - t0); }

__device__ __forceinline__ uint32_t seg_len(const Plan& pl, const Params& p, uint32_t k) {
    return k < pl.whole ? p.n_kv_tiles : (k == pl.whole ? pl.t_len0 : pl.t_len1);
}

// `pl` may be the CTA's copy in shared memory (volatile: the tail fields are then read where they are
// used, once per tail segment, instead of being kept in registers through a role's loops).
template <typename PlanRef>
__device__ __forceinline__ Seg get_seg(PlanRef& pl, uint32_t t0, const Params& p, uint32_t k) {
    Seg s;
    if (k < t0) {
        s.item = blockIdx.x + k * gridDim.x;
        s.j0 = 0;
        s.len = p.n_kv_tiles;
        s.partial = false;
    } else {
        const uint32_t t = k - t0;   // 0 or 1
        s.j0 = t ? 0u : pl.t_j00;
        s.len = t ? pl.t_len1 : pl.t_len0;
        s.item = p.full_rounds * gridDim.x + pl.t_item0 + t;
        s.partial = s.len != p.n_kv_tiles;
    }
    return s;
}

// The CTA whose tail range holds tail key step `step` (ranges are [c*T/tg, (c+1)*T/tg)).
// The launcher only divides a round when T * tg fits in 32 bits.
__device__ __forceinline__ uint32_t tail_cta_of(uint32_t step, uint32_t T, uint32_t tg) {
    return ((step + 1u) * tg - 1u) / T;
}

// ---- a divided work item: hand-over and merge of its parts -------------------------------------
// Scratch of one (slot, tile): H/4 columns of float4, each 128 rows long, so that the 32 lanes of a
// warp (32 consecutive rows) write and read 512 consecutive bytes.  {reference maximum, row sum} of a
// row lie beside it in part_ml.  Indices stay below 2^32 (the whole scratch is a few tens of MB).
template <int H>
__device__ __forceinline__ uint32_t part_o_index(uint32_t slot, uint32_t tile, uint32_t row) {
    return (slot * 2u + tile) * ((H / 4) * kTile) + row;
}

// Rows of O (one per thread: TMEM lane) -> this part's scratch slot, fp32, not normalised.
// `after_last_load` runs once the tile has left TMEM (hand the O columns back there).
template <int H, typename F>
__device__ __forceinline__ void store_part(const Params& p, uint32_t tO, uint32_t slot, uint32_t tile,
                                           uint32_t row, float m, float l, F after_last_load) {
    const uint32_t po = part_o_index<H>(slot, tile, row);
#pragma unroll
    for (int c = 0; c < H / 16; ++c) {
        float o[16];
        tmem_ld16(tO + c * 16, o);
        tmem_wait_ld();
        if (c == H / 16 - 1) after_last_load();
#pragma unroll
        for (int v = 0; v < 4; ++v)
            p.part_o[po + (c * 4 + v) * kTile] = make_float4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
    }
    p.part_ml[(slot * 2u + tile) * kTile + row] = make_float2(m, l);
}

// The parts of tail item `tail_item` are the tail segments of consecutive CTAs c_first ... c_last.
struct PartsOf {
    uint32_t c_first, parts;
};
__device__ __forceinline__ PartsOf parts_of(const Params& p, uint32_t tail_item) {
    const uint32_t n = p.n_kv_tiles, T = p.tail_steps;
    PartsOf r;
    r.c_first = tail_cta_of(tail_item * n, T, p.tail_grid);
    r.parts = min(tail_cta_of(tail_item * n + n - 1u, T, p.tail_grid) - r.c_first + 1u, kMaxParts);
    return r;
}
// Scratch slot of part `pp`: CTA c_first + pp computed it as its first tail segment if that CTA's
// range begins inside this item, else as its second.
__device__ __forceinline__ uint32_t slot_of_part(const Params& p, uint32_t tail_item, uint32_t c_first, uint32_t pp) {
    const uint32_t cta = c_first + pp;
    const uint32_t a = cta * p.tail_steps / p.tail_grid;
    return 2u * cta + (a / p.n_kv_tiles == tail_item ? 0u : 1u);
}

// The common case, two parts: the rows of part `mine` (0 or 1) are in TMEM at tO, the other part is read
// from scratch.  All of the other part is asked for first and `wait_for_o` runs while it is on its way (the
// caller waits there for the last P V if its rows are not complete yet).  Same arithmetic, in the same
// order, as merge_parts.
template <int H, typename F>
__device__ __forceinline__ void merge_two(const Params& p, uint32_t tail_item, uint32_t c_first, uint32_t tile,
                                          uint32_t row, uint32_t mine, uint32_t tO, float m_mine, float l_mine,
                                          __half* y_row, bool row_valid, F wait_for_o) {
    const uint32_t other = slot_of_part(p, tail_item, c_first, 1u - mine);
    const float2 ml_o = __ldcg(p.part_ml + (other * 2u + tile) * kTile + row);
    const float4* src = p.part_o + part_o_index<H>(other, tile, row);
    float4 x[H / 4];
#pragma unroll
    for (int c = 0; c < H / 4; ++c) x[c] = __ldcg(src + c * kTile);
    wait_for_o();
    float m_all = fmaxf(m_mine, ml_o.x);
    if (m_all == -INFINITY) m_all = 0.f;
    const float w_m = ex2_approx((m_mine - m_all) * p.scale_log2);
    const float w_o = ex2_approx((ml_o.x - m_all) * p.scale_log2);
    const bool first = mine == 0u;   // parts are added in the order of the key axis
    const float w0 = first ? w_m : w_o, w1 = first ? w_o : w_m;
    const float inv_l = 1.f / fmaf(w1, first ? ml_o.y : l_mine, fmaf(w0, first ? l_mine : ml_o.y, 0.f));
#pragma unroll
    for (int q = 0; q < H / 32; ++q) {
        float o[32];
        tmem_ld32(tO + q * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float xs[4] = {x[q * 8 + c].x, x[q * 8 + c].y, x[q * 8 + c].z, x[q * 8 + c].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a0 = first ? o[4 * c + e] : xs[e], a1 = first ? xs[e] : o[4 * c + e];
                o[4 * c + e] = fmaf(w1, a1, fmaf(w0, a0, 0.f)) * inv_l;
            }
        }
        if (row_valid) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
                uint4 wv;
                wv.x = pack_half2(o[e], o[e + 1]);
                wv.y = pack_half2(o[e + 2], o[e + 3]);
                wv.z = pack_half2(o[e + 4], o[e + 5]);
                wv.w = pack_half2(o[e + 6], o[e + 7]);
                *reinterpret_cast<uint4*>(y_row + q * 32 + e) = wv;
            }
        }
    }
}

// Add up the parts of 32 rows of one tile of a divided item and write Y.  One thread per row, run by
// a softmax warp (it has the registers to keep a whole row of another part, or half a row of two other
// parts, in flight).  The parts are added in the order of the key axis whoever does the adding, so the
// result does not depend on which part happened to finish last:
//   Y = sum_p w_p O_p / sum_p w_p l_p,   w_p = 2^((m_p - max_q m_q) * scale_log2).
// `mine` is the index of the part whose rows are still in TMEM at tO (with reference m_mine and row
// sum l_mine), or kMaxParts if every part is read from scratch.  An item has two or three parts.
template <int H>
__device__ __forceinline__ void merge_parts(const Params& p, uint32_t tail_item, uint32_t tile, uint32_t row,
                                            uint32_t mine, uint32_t tO, float m_mine, float l_mine,
                                            __half* y_row, bool row_valid) {
    const PartsOf po = parts_of(p, tail_item);
    if (po.parts == 2u && mine < 2u) {
        merge_two<H>(p, tail_item, po.c_first, tile, row, mine, tO, m_mine, l_mine, y_row, row_valid, [] {});
        return;
    }
    uint32_t slot[3];
    float mp[3], lp[3];
#pragma unroll
    for (uint32_t pp = 0; pp < 3; ++pp) {
        slot[pp] = pp < po.parts ? slot_of_part(p, tail_item, po.c_first, pp) : 0u;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (pp < po.parts) ml = pp == mine ? make_float2(m_mine, l_mine) : __ldcg(p.part_ml + (slot[pp] * 2u + tile) * kTile + row);
        mp[pp] = ml.x;
        lp[pp] = ml.y;
    }
    float m_all = fmaxf(fmaxf(mp[0], mp[1]), mp[2]);
    if (m_all == -INFINITY) m_all = 0.f;   // a row masked out in every part: weights 0, Y = 0/0 as torch.softmax gives
    float w[3], l_all = 0.f;
#pragma unroll
    for (uint32_t pp = 0; pp < 3; ++pp) {
        w[pp] = pp < po.parts ? ex2_approx((mp[pp] - m_all) * p.scale_log2) : 0.f;
        if (pp < po.parts) l_all = fmaf(w[pp], lp[pp], l_all);
    }
    const float inv_l = 1.f / l_all;
    if (po.parts == 3u && mine < 3u) {
        // Three parts, one of them in TMEM: half a row of both others in flight at a time.  In key order
        // the parts are (o, a, b), (a, o, b) or (a, b, o) with o the one in TMEM.
        const uint32_t sa = mine == 0u ? slot[1] : slot[0], sb = mine == 2u ? slot[1] : slot[2];
#pragma unroll 1
        for (int half = 0; half < H / 64; ++half) {
            float xa[64], xb[64];
            const float4* pa = p.part_o + part_o_index<H>(sa, tile, row) + (half * 16) * kTile;
            const float4* pb = p.part_o + part_o_index<H>(sb, tile, row) + (half * 16) * kTile;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float4 v = __ldcg(pa + c * kTile);
                xa[4 * c] = v.x; xa[4 * c + 1] = v.y; xa[4 * c + 2] = v.z; xa[4 * c + 3] = v.w;
            }
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float4 v = __ldcg(pb + c * kTile);
                xb[4 * c] = v.x; xb[4 * c + 1] = v.y; xb[4 * c + 2] = v.z; xb[4 * c + 3] = v.w;
            }
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                float o[32];
                tmem_ld32(tO + half * 64 + sub * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float a = xa[sub * 32 + e], bq = xb[sub * 32 + e];
                    const float v0 = mine == 0u ? o[e] : a;
                    const float v1 = mine == 0u ? a : (mine == 1u ? o[e] : bq);
                    const float v2 = mine == 2u ? o[e] : bq;
                    o[e] = fmaf(w[2], v2, fmaf(w[1], v1, fmaf(w[0], v0, 0.f))) * inv_l;
                }
                if (row_valid) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 wv;
                        wv.x = pack_half2(o[e], o[e + 1]);
                        wv.y = pack_half2(o[e + 2], o[e + 3]);
                        wv.z = pack_half2(o[e + 4], o[e + 5]);
                        wv.w = pack_half2(o[e + 6], o[e + 7]);
                        *reinterpret_cast<uint4*>(y_row + half * 64 + sub * 32 + e) = wv;
                    }
                }
            }
        }
        return;
    }
    // Every part from scratch (an epilogue warp's part was the last of its item): half a row of two
    // parts in flight at a time, the third, if there is one, behind them.
#pragma unroll 1
    for (int half = 0; half < H / 64; ++half) {
        float xa[64], xb[64];
        const float4* pa = p.part_o + part_o_index<H>(slot[0], tile, row) + (half * 16) * kTile;
        const float4* pb = p.part_o + part_o_index<H>(slot[1], tile, row) + (half * 16) * kTile;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const float4 v = __ldcg(pa + c * kTile);
            xa[4 * c] = v.x; xa[4 * c + 1] = v.y; xa[4 * c + 2] = v.z; xa[4 * c + 3] = v.w;
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const float4 v = __ldcg(pb + c * kTile);
            xb[4 * c] = v.x; xb[4 * c + 1] = v.y; xb[4 * c + 2] = v.z; xb[4 * c + 3] = v.w;
        }
#pragma unroll
        for (int e = 0; e < 64; ++e) xa[e] = fmaf(w[1], xb[e], fmaf(w[0], xa[e], 0.f));
        if (po.parts > 2u) {
            const float4* pc = p.part_o + part_o_index<H>(slot[2], tile, row) + (half * 16) * kTile;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float4 v = __ldcg(pc + c * kTile);
                xb[4 * c] = v.x; xb[4 * c + 1] = v.y; xb[4 * c + 2] = v.z; xb[4 * c + 3] = v.w;
            }
#pragma unroll
            for (int e = 0; e < 64; ++e) xa[e] = fmaf(w[2], xb[e], xa[e]);
        }
        if (row_valid) {
#pragma unroll
            for (int e = 0; e < 64; e += 8) {
                uint4 wv;
                wv.x = pack_half2(xa[e] * inv_l, xa[e + 1] * inv_l);
                wv.y = pack_half2(xa[e + 2] * inv_l, xa[e + 3] * inv_l);
                wv.z = pack_half2(xa[e + 4] * inv_l, xa[e + 5] * inv_l);
                wv.w = pack_half2(xa[e + 6] * inv_l, xa[e + 7] * inv_l);
                *reinterpret_cast<uint4*>(y_row + half * 64 + e) = wv;
            }
        }
    }
}

// Persistent: grid = min(number of SMs, work items) (the number of SMs when the tail round is
// divided), block = 512.  Every role walks the same list of segments (Plan); the key steps of
// consecutive segments form one continuous sequence of "global steps", so the two-tile ping-pong
// never drains: while the epilogue warps finish segment k, the MMA and softmax warps are already in
// segment k+1.
//
// warps 0-3: softmax of query tile 0; 4-7: softmax of tile 1 (each also rescales its O rows in
// the rare steps whose reference maximum moves); 8-11: epilogue (Y = O / l, or the hand-over and
// merge of a partial segment); 12: MMA issue (one elected lane) and TMEM owner; 13: TMA producer
// (one lane); 14: second MMA issuing warp at H = 128 (12 issues Q K^T, 14 issues P V); 15: idle.
//
// Per tile and key step: Q K^T -> S; the softmax warps read S into registers and say so (SFREE),
// which lets the next Q K^T into the S buffer; they write P into the tile's P columns once the
// previous step's P V has read them (PV); P V accumulates into O.  Nothing of a tile's next Q K^T
// waits for its P V.  With kHasMask the softmax warps add the additive mask row (read with 16-byte
// loads) to the scores they have just read.
//
// Barrier phases (the parity to wait for is the low bit of the index):
//   per global step g:  S_i (MMA -> softmax), SFREE (softmax -> MMA; at H = 128 one barrier whose
//                phase is the use 2g + i of the shared S buffer), P_i (softmax -> MMA),
//                PV_i (MMA -> softmax and, for the segment's last step, epilogue)
//   per segment k:  QFULL_i (TMA -> MMA), QEMPTY_i (MMA -> TMA), A_i (softmax -> epilogue),
//                OFREE_i (epilogue -> MMA and softmax)
//   per ring item t (K0 V0 K1 V1 ... across segments):  FULL[t % NS], EMPTY[t % NS]
//
// Build with -DFA_CYCLES to make CTA 0 record, per launch, the global timer at its entry, after its wait
// for the previous kernel and at its end, and its SM clock count in between, in Params::cycles (a
// diagnostic: the clock count compares versions of the kernel independently of the clock the GPU happens
// to run at, the timer shows the gaps between launches; absent from normal builds).
template <int H, bool kHasMask>
__global__ void __launch_bounds__(512, 1)
fa_fwd_pipelined(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ CUtensorMap tmM, const Params p) {
    using G = TileGeom<H>;
    using C = PipeCfg<H, kHasMask>;
    constexpr int NS = C::kStages;
    enum {
        BAR_QFULL0 = 0, BAR_QFULL1,  // TMA -> MMA: query tile landed
        BAR_QEMPTY0, BAR_QEMPTY1,    // MMA -> TMA: the segment's last Q K^T of this tile has retired
        BAR_S0, BAR_S1,              // MMA -> softmax: S tile complete
        BAR_P0, BAR_P1,              // softmax -> MMA: P written (and O rescaled in the rare steps
                                     // that need it); 4 arrivals, one per softmax warp
        BAR_SFREE0, BAR_SFREE1,      // softmax -> MMA: S read into registers (4 arrivals); with the
                                     // one S buffer of H = 128 only the first, one phase per use
        BAR_PV0, BAR_PV1,            // MMA -> softmax (P buffer free, O at rest) and epilogue: P V complete
        BAR_A0, BAR_A1,              // softmax -> epilogue: final row sums in shared memory (4)
        BAR_OFREE0, BAR_OFREE1,      // epilogue -> MMA, softmax: O tile read out (4 arrivals)
        BAR_EPI,                     // epilogue -> softmax: the epilogue warps are through (4 arrivals)
        BAR_MFULL0, BAR_MFULL1,      // TMA -> softmax of tile i: its mask tile of this key step landed (one buffer,
                                     // filled for the two tiles in turn; a barrier per tile, one phase per key step,
                                     // so that a tile can never take the other tile's phase for its own)
        BAR_MEMPTY0, BAR_MEMPTY1,    // softmax of tile i -> TMA: the mask tile has been read (4 arrivals)
        BAR_FINAL,                   // MMA -> itself: every MMA retired
        BAR_FINAL2,                  // the same for the second issuing warp
        BAR_QB,                      // QFULL0, QFULL1, QEMPTY0, QEMPTY1 of the second query buffer (H = 64)
        BAR_FULL = BAR_QB + 4,       // NS ring barriers TMA -> MMA
        BAR_EMPTY = BAR_FULL + NS,   // NS ring barriers MMA -> TMA
        BAR_COUNT = BAR_EMPTY + NS
    };

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[BAR_COUNT];
    __shared__ float l_buf[2][2][kTile];  // [segment parity][tile][row] final row sums
    __shared__ float m_buf[2][2][kTile];  // ... and the reference maxima they are relative to
    __shared__ uint32_t deferred[2][4];            // [tile][row quarter]: the epilogue warps' part (first of two tail segments) was the last of its item
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_flag;

    const uint32_t tid = threadIdx.x;
#ifdef FA_CYCLES
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) p.cycles[4 * (p.launch_id & 63u)] = global_timer_ns();
#endif
    const uint32_t warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler
    const uint32_t lane = tid & 31u;
    const uint32_t q_pairs = p.q_pairs;
    __shared__ Plan plan_smem;
    volatile Plan& pl_s = plan_smem;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem_base;                   // two tiles per buffer
    const uint32_t sRing = smem_base + C::kQBufs * C::kQBytes;   // NS tiles
    const uint32_t sMask = sRing + C::kRingBytes;    // one mask tile (instances with a mask only)
    const uint32_t sStage = sMask + C::kMaskBytes;   // epilogue staging, 4 KiB per epilogue warp
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };
    // Segment k's query tiles: buffer k mod kQBufs; its barriers complete one phase per use of that buffer.
    auto q_addr = [&](uint32_t k, uint32_t i) { return sQ + (k % C::kQBufs) * C::kQBytes + i * G::kTileBytes; };
    auto q_phase = [&](uint32_t k) { return (k / C::kQBufs) & 1u; };
    auto bar_qfull = [&](uint32_t k, uint32_t i) { return bar(((k % C::kQBufs) ? BAR_QB : BAR_QFULL0) + i); };
    auto bar_qempty = [&](uint32_t k, uint32_t i) { return bar(((k % C::kQBufs) ? BAR_QB + 2 : BAR_QEMPTY0) + i); };
    auto code_qfull = [&](uint32_t k, uint32_t i) { return static_cast<uint32_t>(((k % C::kQBufs) ? BAR_QB : BAR_QFULL0) + i); };
    const WaitCtl ctl{p.status, &abort_flag, kWaitCapCycles, p.status + 2, p.launch_id};

    // What the producer thread asks for first (query tile 0 and the first K tile of the CTA's first segment): worked
    // out here, ahead of the wait for the previous kernel, and asked for straight behind that wait, before the
    // thread has found its way into its role's loop (measured: the first copy goes out ~1000 clocks sooner).
    int32_t first_col0 = 0, first_batch = 0, first_q_row0 = 0, first_key0 = 0;
    bool first_known = false;
    if (tid == 13 * 32) {
        // The plan of this CTA, and a request for the tiles it needs first to be brought into L2.  In a
        // launch that overlaps the previous kernel of the stream this CTA may be here long before that
        // kernel completes; a prefetch returns nothing to the SM, and L2 is where that kernel's writes
        // land, so whatever it still writes is what the loads after the wait below will read.
        const Plan mine = make_plan(p);
        plan_smem = mine;
        if (mine.nseg > 0u) {
            const Seg sg = get_seg(mine, mine.whole, p, 0);
            const uint32_t bh = sg.item / q_pairs;
            const int32_t col0 = static_cast<int32_t>((bh % p.R) * H), batch = static_cast<int32_t>(bh / p.R);
            const int32_t q_row0 = static_cast<int32_t>((sg.item % q_pairs) * 2u * kTile);
            first_col0 = col0, first_batch = batch, first_q_row0 = q_row0, first_key0 = static_cast<int32_t>(sg.j0 * kTile);
            first_known = true;
            prefetch_tile_l2<H>(&tmQ, col0, q_row0, batch);
            prefetch_tile_l2<H>(&tmK, col0, static_cast<int32_t>(sg.j0 * kTile), batch);
            prefetch_tile_l2<H>(&tmQ, col0, q_row0 + kTile, batch);
            prefetch_tile_l2<H>(&tmV, col0, static_cast<int32_t>(sg.j0 * kTile), batch);
            if (sg.len > 1u) {
                prefetch_tile_l2<H>(&tmK, col0, static_cast<int32_t>((sg.j0 + 1u) * kTile), batch);
                prefetch_tile_l2<H>(&tmV, col0, static_cast<int32_t>((sg.j0 + 1u) * kTile), batch);
            }
        }
    }
    if (tid == 0) {
        prefetch_tensormap(&tmY);
#pragma unroll
        for (int i = 0; i < BAR_COUNT; ++i) {
            // one arrival per warp (after __syncwarp), not per thread: 128 arrivals on one
            // shared-memory word serialise
            const bool per_warp = (i == BAR_P0 || i == BAR_P1 || i == BAR_SFREE0 || i == BAR_SFREE1 ||
                                   i == BAR_A0 || i == BAR_A1 || i == BAR_EPI || i == BAR_MEMPTY0 || i == BAR_MEMPTY1 ||
                                   i == BAR_OFREE0 || i == BAR_OFREE1);
            mbar_init(bar(i), per_warp ? 4u : 1u);
        }
        abort_flag = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) (&deferred[0][0])[i] = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
        if constexpr (kHasMask) prefetch_tensormap(&tmM);
    }
#ifdef FA_DEBUG
    dbg_begin(p, ctl, smem_base, C::kSmemBytes - 1024);
#endif
    if (warp == 12) {
        tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
#ifdef FA_DEBUG
    if (tid == 0) dbg_tmem(tmem_slot, C::kTmemCols);
    __syncthreads();
#endif
    // Barriers, TMEM and descriptors are set up; nothing of global memory has been read or written yet.
    // In a launch that was allowed to overlap the previous kernel of the stream, wait here for that
    // kernel to complete, then let the next launch's CTAs take the SMs this grid's CTAs leave (they
    // will stop at this same point: the overlap is never deeper than one launch).
    grid_dep_wait();
    grid_dep_launch();
    if (first_known) {   // the producer thread only
        load_tile<H>(sQ, &tmQ, bar(BAR_QFULL0), first_col0, first_q_row0, first_batch);
        load_tile<H>(sRing, &tmK, bar(BAR_FULL), first_col0, first_key0, first_batch);
    }
    if (tid == 15 * 32) leave_early_if_launch_failed(ctl);   // warp 15 has no other work
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
    const uint32_t nseg = pl_s.nseg, ntail = pl_s.ntail, t0 = nseg - ntail;   // t0: first tail segment
#ifdef FA_CYCLES
    long long cyc0 = 0;
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) {
        p.cycles[4 * (p.launch_id & 63u) + 1] = global_timer_ns();
        cyc0 = clock64();
    }
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
        uint32_t g = 0;   // global step
        float m = -INFINITY, l = 0.f;
        for (uint32_t k = 0; k < nseg; ++k) {
            const Seg sg = get_seg(pl_s, t0, p, k);
            m = -INFINITY;
            l = 0.f;
            // with a mask: the row of mask[batch] this thread adds to its scores
            const __half* mask_row = nullptr;
            uint32_t mask_vec = 2;
            if constexpr (kHasMask) {
                const uint32_t q_row = ((sg.item % q_pairs) * 2u + i) * kTile + row;
                const uint32_t batch = (sg.item / q_pairs) / p.R;
                if (q_row < p.L) mask_row = p.mask + (static_cast<size_t>(batch) * p.L + q_row) * p.L;
                mask_vec = mask_row_alignment(p);
            }
            for (uint32_t jj = 0; jj < sg.len; ++jj, ++g) {
                const uint32_t j = sg.j0 + jj;
                mbar_wait(bar(BAR_S0 + i), g & 1u, ctl, kRoleSoftmax | (BAR_S0 + i));
                tc_fence_after();
                __syncwarp();
                float s[kTile];
                const bool ragged = (j + 1) * kTile > p.L;
                const bool first = jj == 0;
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
                if constexpr (kHasMask) {
                    if (p.mask_tma != 0u) {
                        // The mask tile of this tile and step, brought in by TMA into the one mask buffer; it is
                        // handed back as soon as it has been read.
                        mbar_wait(bar(BAR_MFULL0 + i), g & 1u, ctl, kRoleSoftmax | (BAR_MFULL0 + i));
                        add_mask_tile_row(s, sMask, row, p.mask_to_score);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(BAR_MEMPTY0 + i));
                    } else if (mask_row != nullptr) {
                        add_mask_row(s, mask_row + static_cast<size_t>(j) * kTile,
                                     min(static_cast<int>(p.L - j * kTile), kTile), p.mask_to_score, mask_vec);
                    }
                }
                if (ragged) mask_tail(s, static_cast<int>(p.L - j * kTile));
                if (first) m = row_max(s);   // first key tile of the segment: the reference is its row maximum
                // Exponentials against the standing reference.  The reference only has to move when a score
                // exceeds it by more than 2^8 in the exp2 domain.  P has one buffer per tile and the previous
                // step's P V may still be reading it: the first chunks' exponentials go to registers meanwhile.
                {
                    // A row that has seen nothing but -inf so far (possible only with a mask) takes 0 as
                    // the reference of its exponents, so that P = 0 and l = 0 instead of inf - inf.
                    float nmc = -m * c;
                    if constexpr (kHasMask) nmc = (m == -INFINITY) ? 0.f : nmc;
                    float mx4[4];   // (not used: the row maximum is only taken when the row sum asks for it)
                    uint32_t held[16 * (C::kHeldChunks > 0 ? C::kHeldChunks : 1)];
                    float sum = exp_chunks<0, C::kHeldChunks, false, false>(s, c, nmc, tP, mx4, held);
                    if constexpr (C::kHeldChunks > 0) {
                        if (g > 0) {
                            mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                            tc_fence_after();
                        }
                    }
#pragma unroll
                    for (int ch = 0; ch < C::kHeldChunks; ++ch) tmem_st16(tP + ch * 16, held + ch * 16);
                    sum += exp_chunks<C::kHeldChunks, 4, false>(s, c, nmc, tP, mx4);
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
                        // Some row of this warp needs a new reference: redo the warp's exponentials
                        // (rows that keep theirs reproduce the same P) and rescale O by alpha; the
                        // previous step's P V has retired (waited for above), so O is at rest.
                        const float m_new = moved ? mx : m;
                        const float alpha = moved ? ex2_approx((m - m_new) * c) : 1.f;
                        m = m_new;
                        float nmc2 = -m * c;
                        if constexpr (kHasMask) nmc2 = (m == -INFINITY) ? 0.f : nmc2;
                        float unused[4];
                        l = l * alpha + exp_chunks<0, 4, false>(s, c, nmc2, tP, unused);
                        // (This wait returns at once.  It is here because with a branch point at this
                        // place of the rare path the compiler allocates the common path without spills.)
                        if (g > 0) mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                        tc_fence_after();
                        __syncwarp();
                        if (!first) rescale_o_row<H>(tO, alpha);   // the segment's first P V overwrites O
                    } else {
                        l += sum;
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_P0 + i));
            }
            // Hand the row sums (and the references they are relative to) to the epilogue.  The A
            // barrier may run at most one phase ahead of the epilogue's wait, so the previous segment's
            // O must have been read out first (always true already when a segment has two or more
            // key steps).
            // (With kSoftmaxWritesLast the CTA's last segment is finished by these warps themselves, below.)
            if (!C::kSoftmaxWritesLast || k + 1u < nseg) {
                if (k > 0) mbar_wait(bar(BAR_OFREE0 + i), (k - 1u) & 1u, ctl, kRoleSoftmax | (BAR_OFREE0 + i));
                l_buf[k & 1u][i][row] = l;
                m_buf[k & 1u][i][row] = m;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_A0 + i));
            }
        }
        // ---- the CTA's last segment ---------------------------------------------------------------
        // If this CTA's last segment is a part of a divided item, these warps finish it themselves:
        // they have nothing else left to do, they have the registers to keep many loads in flight, and
        // the part's rows can come straight from TMEM.  A warp that finds every other part of its 32
        // rows already counted in adds the parts up and writes Y; otherwise it leaves its rows in the
        // CTA's scratch slot and counts itself in (and adds up after all if that made it the last).
        const uint32_t wq = warp & 3u;
        bool last_is_whole = C::kSoftmaxWritesLast && nseg > 0u;
        if (ntail > 0u) {   // the CTA's last segment is a tail segment
            const Seg sg = get_seg(pl_s, t0, p, nseg - 1u);
            if (sg.partial) {
                last_is_whole = false;
                const uint32_t tail_item = seg_tail_item(pl_s, t0, nseg - 1u);
                const PartsOf po = parts_of(p, tail_item);
                const uint32_t mine = blockIdx.x - po.c_first;
                uint32_t* cnt = p.part_cnt + (tail_item * 2u + i) * 4u + wq;
                const uint32_t q_row = ((sg.item % q_pairs) * 2u + i) * kTile + row;
                const uint32_t bh = sg.item / q_pairs;
                __half* y_row = p.y + (static_cast<size_t>(bh / p.R) * p.L + q_row) * p.F + (bh % p.R) * H;
                auto wait_for_o = [&] {   // the last P V: this tile's O rows are complete
                    mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
                    tc_fence_after();
                    __syncwarp();
                };
                // The counter is looked at while the last P V is still running.  Parts are counted in only
                // when they are complete, so "every other part is in" stays true once it has been seen.
                uint32_t seen = 0;
                if (lane == 0) seen = ld_acquire_gpu(cnt);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                bool last = seen + 1u == po.parts;
                if (last && po.parts == 2u) {
                    merge_two<H>(p, tail_item, po.c_first, i, row, mine, tO, m, l, y_row, q_row < p.L, wait_for_o);
                } else {
                    wait_for_o();
                    if (!last) {
                        store_part<H>(p, tO, seg_slot(t0, nseg - 1u), i, row, m, l, [] {});
                        __threadfence();    // the part is complete once every lane's stores are visible to the device
                        __syncwarp();
                        uint32_t arrived = 0;
                        if (lane == 0) arrived = atomicAdd(cnt, 1u);
                        arrived = __shfl_sync(0xffffffffu, arrived, 0);
                        last = arrived + 1u == po.parts;
                        if (last) __threadfence();
                    }
                    if (last)
                        merge_parts<H>(p, tail_item, i, row, mine, tO, m, l, y_row, q_row < p.L);
                }
                if (last) {
                    __syncwarp();
                    if (lane == 0) atomicExch(cnt, 0u);   // the counter is left at zero for the next launch
                }
            }
        }
        if constexpr (C::kSoftmaxWritesLast) if (last_is_whole) {
            // A whole work item: nothing is left to overlap its epilogue with, so these warps write Y themselves,
            // both tiles at once (each thread has its row sum, and the registers to take the whole O row in one
            // round trip), instead of handing the two tiles to the four epilogue warps one after the other.
            // Staging area: the tile's own query buffer, which its last Q K^T has long let go of.
            const Seg sg = get_seg(pl_s, t0, p, nseg - 1u);
            const uint32_t bh = sg.item / q_pairs;
            const int32_t row0 = static_cast<int32_t>(((sg.item % q_pairs) * 2u + i) * kTile + wq * 32u);
            const uint32_t stage = q_addr(nseg - 1u, i) + wq * static_cast<uint32_t>((H / 64) * 4096);
            mbar_wait(bar(BAR_PV0 + i), (g - 1u) & 1u, ctl, kRoleSoftmax | (BAR_PV0 + i));
            tc_fence_after();
            __syncwarp();
            stage_o_row<H>(tO, 1.f / l, stage, lane);
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
        // A part that the epilogue warps put into scratch (the first tail segment of a CTA that has two) and
        // that turned out to be the last of its item: added up here, every part read from scratch.
        if (ntail == 2u) {
            mbar_wait_relaxed(bar(BAR_EPI), 0, ctl, kRoleSoftmax | BAR_EPI, 100);
            if (deferred[i][wq] != 0u) {
                const Seg sg = get_seg(pl_s, t0, p, t0);
                const uint32_t q_row = ((sg.item % q_pairs) * 2u + i) * kTile + row;
                const uint32_t bh = sg.item / q_pairs;
                __half* y_row = p.y + (static_cast<size_t>(bh / p.R) * p.L + q_row) * p.F + (bh % p.R) * H;
                const uint32_t tail_item = seg_tail_item(pl_s, t0, t0);
                __threadfence();
                merge_parts<H>(p, tail_item, i, row, kMaxParts, tO, 0.f, 0.f, y_row, q_row < p.L);
                __syncwarp();
                if (lane == 0) atomicExch(p.part_cnt + (tail_item * 2u + i) * 4u + wq, 0u);
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ epilogue
        // Each warp owns 32 rows of the tile.
        // Whole item: it reads them from TMEM, scales by 1/l, rounds to fp16 and writes 16-byte vectors
        // into its 4 KiB staging buffer (rows of 128 bytes, 128-byte swizzle), which one TMA store
        // sends to Y: the warp is not held up by scattered global stores and the O tile is handed
        // back as soon as it is in registers.
        // Part of a divided item that is not the CTA's last segment: the rows go to this CTA's scratch
        // slot as they are (fp32, not normalised) together with (reference maximum, row sum), and the
        // warp counts itself in on the item's counter (see store_part, merge_parts).
        setmaxnreg_dec<64>();
        const uint32_t row = tid & 127u;
        const uint32_t wq = warp & 3u;
        const uint32_t lane_off = (wq * 32u) << 16;
        const uint32_t stage = sStage + wq * 4096u;
        uint32_t g_end = 0;   // global steps up to and including the current segment
        for (uint32_t k = 0; k < nseg; ++k) {
            const Seg sg = get_seg(pl_s, t0, p, k);
            // the softmax warps finish a final part themselves, and with kSoftmaxWritesLast a final whole item too
            if (k + 1u == nseg && (sg.partial || C::kSoftmaxWritesLast)) break;
            g_end += sg.len;
            const uint32_t q_pair = sg.item % q_pairs, bh = sg.item / q_pairs;
            const uint32_t head = bh % p.R, batch = bh / p.R;
#pragma unroll
            for (uint32_t i = 0; i < 2; ++i) {
                // this wait lasts for a whole segment: poll every 100 ns
                mbar_wait_relaxed(bar(BAR_A0 + i), k & 1u, ctl, kRoleEpilogue | (BAR_A0 + i), 100);
                const float l_row = l_buf[k & 1u][i][row];
                // The segment's last P V of this tile.  Every earlier phase of this barrier has
                // completed by the time the softmax warps signalled and the next phase needs this
                // epilogue's OFREE arrival, so the parity test is unambiguous.
                mbar_wait(bar(BAR_PV0 + i), (g_end - 1u) & 1u, ctl, kRoleEpilogue | (BAR_PV0 + i));
                tc_fence_after();
                __syncwarp();
                const uint32_t tO = tmem_base + lane_off + (i ? C::kColO1 : C::kColO0);
                const int32_t row0 = static_cast<int32_t>((q_pair * 2u + i) * kTile + wq * 32u);
                if (!sg.partial) {
                    const float inv_l = 1.f / l_row;
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
                                st_shared_v4(stage + lane * 128u + chunk * 16u, w0, w1, w2, w3);
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
                } else {
                    // A tail segment that is not the CTA's last segment: the rows go to the scratch slot as
                    // they are and the O tile is handed back.
                    store_part<H>(p, tO, seg_slot(t0, k), i, row, m_buf[k & 1u][i][row], l_row, [&] {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(BAR_OFREE0 + i));
                    });
                }
            }
            if (sg.partial) {
                // Both O tiles have been handed back (the next segment's P V are not held up by what
                // follows).  Once every lane's stores are visible to the device the warp counts itself in
                // on the item's two counters.  If that makes its part the last of the item, the softmax warp
                // of these rows adds the parts up at the end of the kernel (it has the registers to do it in
                // a few trips to L2, and by then every part has long been complete).
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    const uint32_t tail_item = seg_tail_item(pl_s, t0, k);
                    const PartsOf po = parts_of(p, tail_item);
#pragma unroll
                    for (uint32_t i = 0; i < 2; ++i)
                        if (atomicAdd(p.part_cnt + (tail_item * 2u + i) * 4u + wq, 1u) + 1u == po.parts)
                            deferred[i][wq] = 1u;
                }
            }
            // the one tail segment this role takes is through: the softmax warps may look at the flags
            if (sg.partial) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_EPI));
            }
        }
        // The staging buffers must have been read before the CTA gives up its shared memory; the writes
        // to Y themselves are complete, like every other write, when the grid is.
        if (lane == 0) bulk_wait_read_all();
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
            auto mwait = [&](uint32_t b, uint32_t parity, uint32_t code) {
                ok &= mbar_wait(b, parity, ctl, kRoleMma | code);
            };
            auto wait_full = [&](uint32_t t) { mwait(bar(BAR_FULL + (t % NS)), (t / NS) & 1u, BAR_FULL + (t % NS)); };
            auto free_slot = [&](uint32_t t) { tc_commit(bar(BAR_EMPTY + (t % NS))); };
            Plan pl;   // this role keeps the plan in registers: it may not wait for shared memory between MMAs
            pl.ntail = ntail; pl.whole = t0; pl.nseg = nseg; pl.steps = pl_s.steps; pl.t_item0 = 0; pl.t_j00 = 0;
            pl.t_len0 = pl_s.t_len0; pl.t_len1 = pl_s.t_len1;
            const uint32_t steps = pl.steps;   // global steps of this CTA
            // ring item 2g is the K tile of global step g, item 2g+1 its V tile
            // (k, j, len): segment of the step a loop is working on, its position in it, its length
            uint32_t k = 0, j = 0, len = seg_len(pl, p, 0);
            if (steps > 0 && warp == 12) {
                // S tiles of the very first step
                mwait(bar_qfull(0, 0), 0, code_qfull(0, 0));
                wait_full(0);
                tc_fence_after();
                if (leader && ok) {
                    issue_qk<H>(tS0, q_addr(0, 0), slot_addr(0));
                    tc_commit(bar(BAR_S0));
                    if (len == 1) tc_commit(bar_qempty(0, 0));
                }
                mwait(bar_qfull(0, 1), 0, code_qfull(0, 1));
                // one S buffer for both tiles: tile 0's scores must have been read first
                if constexpr (C::kSharedS) mwait(bar(BAR_SFREE0), 0, BAR_SFREE0);
                tc_fence_after();
                if (leader && ok) {
                    issue_qk<H>(tS1, q_addr(0, 1), slot_addr(0));
                    tc_commit(bar(BAR_S1));
                    if (len == 1) tc_commit(bar_qempty(0, 1));
                    free_slot(0);
                }
            }
            if constexpr (C::kTwoIssuers) {
                mbar_poll_declare();
                bool polled = false;
                if (warp == 12) {
                    // Q K^T stream: the scores of step q = 1, 2, ..., tile 0 then tile 1, each as soon as the
                    // softmax warps have read what the S buffer holds.  That K has landed is known long
                    // before; it is tested ahead of the previous step's last MMAs and the answer read
                    // after them (mbar_poll_begin).
                    for (uint32_t q = 1; q < steps; ++q) {
                        bool new_seg = false;            // step q opens segment k
                        if (++j == len) { j = 0; ++k; len = seg_len(pl, p, k); new_seg = true; }
                        const bool last_of_seg = j + 1 == len;   // a segment's last Q K^T is its last use of the query tile
                        const uint32_t tk = 2 * q;
                        if (!(polled && mbar_poll_end<0>())) wait_full(tk);
                        if (new_seg) mwait(bar_qfull(k, 0), q_phase(k), code_qfull(k, 0));
                        // With one S buffer its uses are numbered 2q + i (tile i, step q) and use u
                        // needs the reading of use u - 1 (one barrier, phase = use).
                        mwait(bar(BAR_SFREE0), 1u, BAR_SFREE0);
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS0, q_addr(k, 0), slot_addr(tk));
                            tc_commit(bar(BAR_S0));
                            if (last_of_seg) tc_commit(bar_qempty(k, 0));
                        }
                        if (new_seg) mwait(bar_qfull(k, 1), q_phase(k), code_qfull(k, 1));
                        mwait(bar(BAR_SFREE0), 0u, BAR_SFREE0);
                        tc_fence_after();
                        polled = q + 1 < steps;
                        if (polled) {
                            const uint32_t nk = tk + 2;
                            mbar_poll_begin<0>(bar(BAR_FULL + (nk % NS)), (nk / NS) & 1u);
                        }
                        if (leader && ok) {
                            issue_qk<H>(tS1, q_addr(k, 1), slot_addr(tk));
                            tc_commit(bar(BAR_S1));
                            if (last_of_seg) tc_commit(bar_qempty(k, 1));
                            free_slot(tk);
                        }
                    }
                } else {
                    // P V stream: for every step the products of tile 0 and tile 1 as their P arrive.
                    for (uint32_t g = 0; g < steps; ++g) {
                        const uint32_t tv = 2 * g + 1;
                        const uint32_t acc = j > 0 ? 1u : 0u;
                        if (!(polled && mbar_poll_end<1>())) wait_full(tv);
                        if (j == 0 && k > 0) mwait(bar(BAR_OFREE0), (k - 1u) & 1u, BAR_OFREE0);
                        mwait(bar(BAR_P0), g & 1u, BAR_P0);
                        tc_fence_after();
                        if (leader && ok) {
                            issue_pv<H>(tO0, tP0, slot_addr(tv), acc);
                            tc_commit(bar(BAR_PV0));
                        }
                        if (j == 0 && k > 0) mwait(bar(BAR_OFREE1), (k - 1u) & 1u, BAR_OFREE1);
                        mwait(bar(BAR_P1), g & 1u, BAR_P1);
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
                        if (++j == len) { j = 0; ++k; len = seg_len(pl, p, k); }
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
                    const bool more = g + 1 < steps;            // a next global step exists
                    const bool next_new_seg = j + 1 == len;     // ... and it opens segment k + 1
                    // is the next step the last of its segment (its Q K^T the last use of the query tile)?
                    const bool next_last_of_seg = next_new_seg ? seg_len(pl, p, k + 1u) == 1u : j + 2 == len;
                    const uint32_t acc = j > 0 ? 1u : 0u;
                    const uint32_t kn = next_new_seg ? k + 1u : k;   // the segment of the next step
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
                            if (next_new_seg) mwait(bar_qfull(kn, 0), q_phase(kn), code_qfull(kn, 0));
                            if (!ok_s0) mwait(bar(BAR_SFREE0), g & 1u, BAR_SFREE0);
                        }
                    }
                    if (j == 0 && k > 0) mwait(bar(BAR_OFREE0), (k - 1u) & 1u, BAR_OFREE0);
                    // tile 0
                    if (more) {
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS0, q_addr(kn, 0), slot_addr(tk));
                            tc_commit(bar(BAR_S0));
                            if (next_last_of_seg) tc_commit(bar_qempty(kn, 0));
                        }
                    }
                    mwait(bar(BAR_P0), g & 1u, BAR_P0);
                    tc_fence_after();
                    if (more) mbar_poll_begin<3>(bar(BAR_SFREE1), g & 1u);   // read behind the P V below
                    if (leader && ok) {
                        issue_pv<H>(tO0, tP0, slot_addr(tv), acc);
                        tc_commit(bar(BAR_PV0));
                    }
                    // tile 1
                    if (more && next_new_seg) mwait(bar_qfull(kn, 1), q_phase(kn), code_qfull(kn, 1));
                    if (j == 0 && k > 0) mwait(bar(BAR_OFREE1), (k - 1u) & 1u, BAR_OFREE1);
                    if (more) {
                        if (!mbar_poll_end<3>()) mwait(bar(BAR_SFREE1), g & 1u, BAR_SFREE1);
                        tc_fence_after();
                        if (leader && ok) {
                            issue_qk<H>(tS1, q_addr(kn, 1), slot_addr(tk));
                            tc_commit(bar(BAR_S1));
                            if (next_last_of_seg) tc_commit(bar_qempty(kn, 1));
                            free_slot(tk);
                        }
                    }
                    mwait(bar(BAR_P1), g & 1u, BAR_P1);
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
                    if (++j == len) { j = 0; ++k; len = seg_len(pl, p, k); }
                }
            }
            // Every MMA this warp issued has to retire before the CTA releases tensor memory and shared
            // memory, whether or not a wait gave up on the way: this wait does not look at the abort flag.
            const int bar_final = warp == 12 ? BAR_FINAL : BAR_FINAL2;
            if (leader) tc_commit(bar(bar_final));
            __syncwarp();
            mbar_wait_certain(bar(bar_final), 0, ctl, kRoleMma | static_cast<uint32_t>(bar_final));
        } else if (warp == 13 && elect_one()) {
            // -------------------------------------------------------------- TMA producer
            uint32_t t = 0;           // ring item
            uint32_t k = 0;           // segment
            bool stop = false;
            uint32_t q_asked[2] = {0, 0};   // for how many segments query tile tt has been asked for
            for (; k < nseg && !stop; ++k) {
                const Seg sg = get_seg(pl_s, t0, p, k);
#ifdef FA_DEBUG
                if (!dbg_ok(sg.item < p.n_items && sg.len >= 1u && sg.j0 + sg.len <= p.n_kv_tiles &&
                            (k < t0 || (seg_slot(t0, k) < p.part_slots && seg_tail_item(pl_s, t0, k) < p.tail_items)),
                            kDbgPlan)) break;
#endif
                const uint32_t q_pair = sg.item % q_pairs, bh = sg.item / q_pairs;
                const int32_t col0 = static_cast<int32_t>((bh % p.R) * H);
                const int32_t batch = static_cast<int32_t>(bh / p.R);
                const int32_t q_row0 = static_cast<int32_t>(q_pair * 2u * kTile);
                for (uint32_t tt = 0; tt < 2 * sg.len; ++tt, ++t) {
                    const bool asked_already = t == 0u;   // query tile 0 and K tile 0 of the first segment: see above
                    if (tt < 2) {
                        // query tile tt of this segment, once the buffer's previous user has let go of it
                        if (k >= static_cast<uint32_t>(C::kQBufs) &&
                            !mbar_wait(bar_qempty(k, tt), q_phase(k - C::kQBufs), ctl,
                                       kRoleProducer | (BAR_QEMPTY0 + tt))) { stop = true; break; }
                        if (!asked_already)
                            load_tile<H>(q_addr(k, tt), &tmQ, bar_qfull(k, tt), col0,
                                         q_row0 + static_cast<int32_t>(tt * kTile), batch);
                        q_asked[tt] = k + 1u;
                    }
                    const uint32_t slot = t % NS;
                    if (!mbar_wait(bar(BAR_EMPTY + slot), ((t / NS) & 1u) ^ 1u, ctl,
                                   kRoleProducer | (BAR_EMPTY + slot))) { stop = true; break; }
                    if (!asked_already)
                        load_tile<H>(sRing + slot * G::kTileBytes, (tt & 1u) ? &tmV : &tmK, bar(BAR_FULL + slot),
                                     col0, static_cast<int32_t>((sg.j0 + (tt >> 1)) * kTile), batch);
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
                // the query tiles asked for last (with two buffers, those of the last two segments)
                for (uint32_t tt = 0; tt < 2; ++tt) {
                    const uint32_t first_q = q_asked[tt] > static_cast<uint32_t>(C::kQBufs) ? q_asked[tt] - C::kQBufs : 0u;
                    for (uint32_t kk = first_q; kk < q_asked[tt]; ++kk) {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(bar_qfull(kk, tt), q_phase(kk)) && clock64() - t0 < 200000000LL) {
                        }
                    }
                }
            }
        } else if (kHasMask && warp == 15 && p.mask_tma != 0u && elect_one()) {
            // -------------------------------------------------------------- TMA producer of the mask tiles
            // One buffer, filled for tile 0 and tile 1 of every key step in turn, each time as soon as the softmax
            // warps of the tile before have read it: tile 1 of step g follows tile 0 of step g, tile 0 of step g
            // follows tile 1 of step g - 1.  Boxes that lie beyond the end of the sequence (keys or rows) arrive
            // as zeros.
            uint32_t g = 0;   // global step
            uint32_t asked[2] = {0, 0};   // for how many key steps tile i's mask tile has been asked for
            bool stop = false;
            for (uint32_t k = 0; k < nseg && !stop; ++k) {
                const Seg sg = get_seg(pl_s, t0, p, k);
                const int32_t batch = static_cast<int32_t>((sg.item / q_pairs) / p.R);
                const int32_t q_row0 = static_cast<int32_t>((sg.item % q_pairs) * 2u * kTile);
                for (uint32_t jj = 0; jj < sg.len && !stop; ++jj, ++g) {
                    const int32_t key0 = static_cast<int32_t>((sg.j0 + jj) * kTile);
                    for (uint32_t i = 0; i < 2; ++i) {
                        bool ok = true;
                        if (i == 1) ok = mbar_wait(bar(BAR_MEMPTY0), g & 1u, ctl, kRoleProducer | BAR_MEMPTY0);
                        else if (g > 0) ok = mbar_wait(bar(BAR_MEMPTY1), (g - 1u) & 1u, ctl, kRoleProducer | BAR_MEMPTY1);
                        if (!ok) {
                            stop = true;
                            break;
                        }
                        mbar_expect_tx(bar(BAR_MFULL0 + i), C::kMaskBytes);
                        tma_load_3d(sMask, &tmM, bar(BAR_MFULL0 + i), key0, q_row0 + static_cast<int32_t>(i * kTile), batch);
                        tma_load_3d(sMask + kTile * 128, &tmM, bar(BAR_MFULL0 + i), key0 + 64,
                                    q_row0 + static_cast<int32_t>(i * kTile), batch);
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

    tc_fence_before();
    __syncthreads();
#ifdef FA_CYCLES
    if (p.cycles != nullptr && blockIdx.x == 0 && tid == 0) {
        p.cycles[4 * (p.launch_id & 63u) + 2] = global_timer_ns();
        p.cycles[4 * (p.launch_id & 63u) + 3] = static_cast<unsigned long long>(clock64() - cyc0);
    }
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

#ifdef FA_DEBUG
// Self-test of the checked build's predicates: no copy and no tensor-memory access is made here; the
// predicates are asked about operands that are in order and about operands that are not, and must accept
// the former, refuse the latter and report the first refusal.  status[3] receives one bit per answer.
__global__ void fa_selftest_debug_checks(uint32_t* status) {
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        g_dbg.smem_lo = 0x4000;
        g_dbg.smem_hi = 0x4000 + 64 * 1024;
        g_dbg.F = 512;
        g_dbg.L = 300;
        g_dbg.B = 2;
        g_dbg.tmem_base = 0;
        g_dbg.tmem_cols = 256;
        g_dbg.ctl = WaitCtl{status, &abort_flag, 1000, nullptr, 0};
        uint32_t bits = 0;
        bits |= dbg_copy_ok(0x4000, 4096, 64, 128, 1, false) ? 1u : 0u;          // in order
        bits |= dbg_copy_ok(0x4000 + 1024, 4096, 64, 299, 0, true) ? 2u : 0u;    // in order (a store at the last row)
        bits |= dbg_tmem_ok(128u, 32u) ? 4u : 0u;                                // in order (warp 0, lanes 0-31)
        bits |= dbg_copy_ok(0x4000, 4096, 68, 0, 0, false) ? 0u : 8u;            // x not a multiple of 8: refused first
        bits |= dbg_copy_ok(0x4000 + 62 * 1024, 4096, 0, 0, 0, false) ? 0u : 16u;   // runs past the tile area
        bits |= dbg_copy_ok(0x4000 + 512, 4096, 0, 0, 0, false) ? 0u : 32u;      // not on a 1024-byte boundary
        bits |= dbg_copy_ok(0x4000, 4096, 0, 300, 0, true) ? 0u : 64u;           // a store beyond the last row
        bits |= dbg_copy_ok(0x4000, 4096, 0, -1, 0, true) ? 0u : 128u;           // a store at a negative row
        bits |= dbg_copy_ok(0x4000, 4096, 0, 0, 2, false) ? 0u : 256u;           // batch entry outside the tensor
        bits |= dbg_tmem_ok(240u, 32u) ? 0u : 512u;                              // columns beyond the allocation
        bits |= dbg_tmem_ok((32u << 16) | 0u, 16u) ? 0u : 1024u;                 // another warp's lanes
        status[3] = bits;
    }
}
#endif

}  // namespace fa
