// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, each CTA fetching its own tiles), tcgen05 (TMEM alloc, MMA, ld/st, commit).
// Nothing here is specific to attention.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace fa {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a converged warp (all 32 lanes must execute this together).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .b32 rx;\n\t"
        ".reg .pred px;\n\t"
        "elect.sync rx|px, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, px;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Deferred barrier test for the thread that issues tcgen05.mma.  A shared-memory result reaches that
// thread only behind the MMAs it has queued (150 to 300 clocks during which it issues nothing), even
// when the phase it asks about completed long ago.  For barriers that are known to complete early it
// therefore asks ahead of a group of MMAs and looks at the answer after issuing them:
//   mbar_poll_declare()        once, at the top of the role's code (declares the predicate registers)
//   mbar_poll_begin<N>(...)    mbarrier.test_wait into predicate N; nothing waits for the result yet
//   ... issue a group of MMAs ...
//   mbar_poll_end<N>()         reads predicate N: non-zero if the phase was complete when tested
// The predicates are PTX registers of function scope shared by these pieces of inline assembly, since
// inline assembly cannot hand a predicate to C++.
__device__ __forceinline__ void mbar_poll_declare() {
    asm volatile(".reg .pred fa_poll0, fa_poll1, fa_poll2, fa_poll3;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void mbar_poll_begin(uint32_t bar, uint32_t parity) {
    static_assert(N >= 0 && N < 4, "four predicates are declared");
    if (N == 0) asm volatile("mbarrier.test_wait.parity.shared::cta.b64 fa_poll0, [%0], %1;" ::"r"(bar), "r"(parity) : "memory");
    if (N == 1) asm volatile("mbarrier.test_wait.parity.shared::cta.b64 fa_poll1, [%0], %1;" ::"r"(bar), "r"(parity) : "memory");
    if (N == 2) asm volatile("mbarrier.test_wait.parity.shared::cta.b64 fa_poll2, [%0], %1;" ::"r"(bar), "r"(parity) : "memory");
    if (N == 3) asm volatile("mbarrier.test_wait.parity.shared::cta.b64 fa_poll3, [%0], %1;" ::"r"(bar), "r"(parity) : "memory");
}
template <int N>
__device__ __forceinline__ uint32_t mbar_poll_end() {
    uint32_t ok;
    if (N == 0) asm volatile("selp.u32 %0, 1, 0, fa_poll0;" : "=r"(ok)::"memory");
    if (N == 1) asm volatile("selp.u32 %0, 1, 0, fa_poll1;" : "=r"(ok)::"memory");
    if (N == 2) asm volatile("selp.u32 %0, 1, 0, fa_poll2;" : "=r"(ok)::"memory");
    if (N == 3) asm volatile("selp.u32 %0, 1, 0, fa_poll3;" : "=r"(ok)::"memory");
    return ok;
}

// Where a bounded wait reports: a device status block and a CTA-wide abort flag.
struct WaitCtl {
    uint32_t* status;              // global: [0] first failure code, [1] number of reporting CTAs
    volatile uint32_t* abort_flag; // shared: non-zero once any wait of this CTA has expired
    long long cap_cycles;          // how long one wait may spin
    uint32_t* launch_word;         // global, may be null: receives launch_id when a wait expires, so that
    uint32_t launch_id;            // CTAs of the same launch that start later leave at once
};

// About two seconds at 2 GHz; a whole launch of the largest supported problem takes milliseconds.
constexpr long long kWaitCapCycles = 4000000000LL;

__device__ __forceinline__ void wait_expired(const WaitCtl& ctl, uint32_t code) {
    if (atomicExch(const_cast<uint32_t*>(ctl.abort_flag), 1u) == 0u) {
        atomicCAS(ctl.status, 0u, code);
        atomicAdd(ctl.status + 1, 1u);
        if (ctl.launch_word != nullptr) atomicExch(ctl.launch_word, ctl.launch_id);
    }
}

// A CTA that starts after another CTA of its own launch has given up does not wait for anything:
// it sets its abort flag, runs through its loops and leaves (one thread calls this, no barrier needed:
// the flag is only read on the slow path of a wait).
__device__ __forceinline__ void leave_early_if_launch_failed(const WaitCtl& ctl) {
    if (ctl.launch_word != nullptr &&
        *reinterpret_cast<volatile uint32_t*>(ctl.launch_word) == ctl.launch_id)
        *ctl.abort_flag = 1u;
}

__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, WaitCtl ctl,
                                            uint32_t code) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u) {
            if (*ctl.abort_flag != 0u) return false;
            if (clock64() - t0 > ctl.cap_cycles) {
                wait_expired(ctl, code);
                return false;
            }
        }
    }
    return true;
}

// Same wait for roles that are far from the critical path: sleeps between polls so that the
// polling warp leaves the issue slots of its sub-partition to the warps that are computing.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, WaitCtl ctl,
                                                  uint32_t code, uint32_t sleep_ns) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(sleep_ns);
        if (*ctl.abort_flag != 0u) return false;
        if (clock64() - t0 > ctl.cap_cycles) {
            wait_expired(ctl, code);
            return false;
        }
    }
    return true;
}

// Wait for the phase with the given parity to complete.  Never spins for ever: after the cap (or
// once another wait of this CTA has expired) it returns false and the caller carries on, so that
// every role still reaches the end of the kernel and TMEM is released.  Results are then garbage
// and the status word says so.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, WaitCtl ctl,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctl, code);
}

// Wait for a completion that is certain to come, such as the retirement of MMAs that have been
// issued (tcgen05.commit): it does NOT return early when the CTA's abort flag is set, because the
// caller is about to release what those operations still use (tensor memory, shared memory).  It
// has the same cap as every other wait.
__device__ __forceinline__ bool mbar_wait_certain(uint32_t bar, uint32_t parity, WaitCtl ctl,
                                                  uint32_t code) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u && clock64() - t0 > ctl.cap_cycles) {
            wait_expired(ctl, code);
            return false;
        }
    }
    return true;
}

// ----------------------------------------------------------------------------- checked build (-DFA_DEBUG)
// With -DFA_DEBUG every TMA copy and every tensor-memory access of the kernels checks its operands first:
// the shared-memory side lies inside the CTA's tile area and on a 1024-byte boundary, the innermost
// coordinate is a multiple of 8 elements (16 bytes) and all coordinates lie inside the tensor, a store does
// not start at a negative or out-of-range row, a tensor-memory access stays inside the CTA's allocation and
// on the lanes of the issuing warp.  A failed check records kRoleDebug | <what> in the device status word,
// sets the CTA's abort flag and SKIPS the access (nothing faults; the bounded waits then return at once and
// the CTA leaves).  The kernels also fill their tile area with NaN before the first copy, and the launcher
// fills Y with NaN before the launch, so that anything consumed before it has landed, or never written,
// shows in the result.  Normal builds contain none of this.
#ifdef FA_DEBUG
constexpr uint32_t kRoleDebug = 0x700u;
enum : uint32_t {
    kDbgSmemRange = 1,   // shared-memory operand of a copy outside the tile area
    kDbgSmemAlign,       // ... not on a 1024-byte boundary
    kDbgTmaX,            // innermost coordinate not a multiple of 8 elements
    kDbgTmaCoord,        // a coordinate outside the tensor
    kDbgStoreRow,        // a store starting at a negative row or beyond the last row
    kDbgTmemCols,        // tensor-memory columns outside the allocation
    kDbgTmemLanes,       // tensor-memory lanes that are not the issuing warp's
    kDbgPlan             // a work item, key step or scratch slot outside its range
};
struct DbgCtx {
    uint32_t smem_lo, smem_hi;   // the CTA's tile area in shared memory (shared-window addresses)
    uint32_t F, L, B;            // extent of the tensors in elements / rows / batch entries
    uint32_t tmem_base, tmem_cols;
    WaitCtl ctl;
};
__shared__ DbgCtx g_dbg;   // one per CTA, filled by one thread of each kernel before anything is checked

__device__ __forceinline__ bool dbg_ok(bool cond, uint32_t what) {
    if (!cond) wait_expired(g_dbg.ctl, kRoleDebug | what);
    return cond;
}
// (the innermost extent is F for Q, K, V, Y and L for the mask: a copy whose x lies below max(F, L) passes here)
__device__ __forceinline__ bool dbg_copy_ok(uint32_t saddr, uint32_t bytes, int32_t x, int32_t y, int32_t z, bool store) {
    bool ok = dbg_ok(saddr >= g_dbg.smem_lo && saddr + bytes <= g_dbg.smem_hi, kDbgSmemRange);
    ok &= dbg_ok((saddr & 1023u) == 0u, kDbgSmemAlign);
    ok &= dbg_ok((x & 7) == 0, kDbgTmaX);
    const uint32_t x_extent = (g_dbg.F > g_dbg.L ? g_dbg.F : g_dbg.L) + (store ? 0u : 128u);   // a load may start in the zero fill
    ok &= dbg_ok(x >= 0 && static_cast<uint32_t>(x) < x_extent && z >= 0 && static_cast<uint32_t>(z) < g_dbg.B, kDbgTmaCoord);
    if (store) ok &= dbg_ok(y >= 0 && static_cast<uint32_t>(y) < g_dbg.L, kDbgStoreRow);
    else ok &= dbg_ok(y >= 0, kDbgTmaCoord);   // a load may run past the last row (zero fill), never start before the first
    return ok;
}
__device__ __forceinline__ bool dbg_tmem_ok(uint32_t taddr, uint32_t ncols) {
    const uint32_t col = taddr & 0xFFFFu, base = g_dbg.tmem_base & 0xFFFFu;
    bool ok = dbg_ok(col >= base && col + ncols <= base + g_dbg.tmem_cols, kDbgTmemCols);
    ok &= dbg_ok(((taddr >> 16) & 0x7Fu) == ((threadIdx.x >> 5) & 3u) * 32u, kDbgTmemLanes);
    return ok;
}
#define FA_DBG_COPY(saddr, bytes, x, y, z, store) if (!dbg_copy_ok(saddr, bytes, x, y, z, store)) return
#define FA_DBG_TMEM(taddr, ncols) if (!dbg_tmem_ok(taddr, ncols)) return
#else
#define FA_DBG_COPY(saddr, bytes, x, y, z, store) do {} while (0)
#define FA_DBG_TMEM(taddr, ncols) do {} while (0)
#endif

// ----------------------------------------------------------------------------- launch overlap
// Programmatic dependent launch.  A kernel launched with the "programmatic stream serialization"
// attribute may become resident while the kernel before it in the stream is still running;
// grid_dep_wait() then blocks until that kernel has completed and its writes are visible (it
// returns at once in a launch without the attribute).  grid_dep_launch() tells the scheduler that
// the kernel after this one may be made resident as SMs fall free; it fires once every CTA of
// this grid has executed it.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ----------------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 3-D tiled load global -> shared (this CTA's own shared memory), completion on an mbarrier.
// x is the innermost coordinate; x * sizeof(element) must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar, int32_t x,
                                            int32_t y, int32_t z) {
    FA_DBG_COPY(dst, 4096u, x, y, z, false);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Ask for a tile to be brought into L2 (nothing is returned to the SM and nothing signals completion).
__device__ __forceinline__ void tma_prefetch_l2_3d(const void* map, int32_t x, int32_t y, int32_t z) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(x), "r"(y), "r"(z)
                 : "memory");
}

// 3-D tiled store shared -> global as one bulk group; the box is clipped at the tensor's bounds.
// Coordinates must not be negative; x * sizeof(element) must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_3d(const void* map, uint32_t src, int32_t x, int32_t y, int32_t z) {
    FA_DBG_COPY(src, 4096u, x, y, z, true);
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// every bulk group of this thread has finished READING shared memory (the source may be reused)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// every bulk group of this thread is complete (the global writes are done)
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t (&w)[4]) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
}
__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// The mbarrier receives one arrival when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem];  accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor for kind::f16 with fp16 A and B, fp32 D, M = 128.
// Bits: [4,6) D format (1 = f32); [7,10) A format (0 = f16); [10,13) B format; 15 A major;
// 16 B major (0 = K-major, 1 = MN-major); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t n, uint32_t b_mn_major) {
    return (1u << 4) | (b_mn_major << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// Shared-memory matrix descriptor.  Bits: [0,14) address >> 4; [16,30) leading byte offset >> 4;
// [32,46) stride byte offset >> 4; [46,48) version = 1; [61,64) swizzle (2 = 128 B, 4 = 64 B,
// 6 = 32 B).  `swz` is the swizzle span in bytes, which here is also the pitch of one row.
template <int kSwz>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes) {
    constexpr uint64_t layout = kSwz == 128 ? 2ull : (kSwz == 64 ? 4ull : 6ull);
    constexpr uint64_t sbo = (8ull * kSwz) >> 4;  // eight rows of one swizzle span
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) |
           (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) | (sbo << 32) | (1ull << 46) |
           (layout << 61);
}

// 32 lanes x 32 columns of 32-bit cells: thread t of the warp receives lane (base lane + t),
// register i holds column (base column + i).  A warp may only touch lanes [32*(warp%4), +32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    FA_DBG_TMEM(taddr, 32u);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]),
          "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]),
          "=f"(v[14]), "=f"(v[15]), "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]),
          "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]), "=f"(v[25]),
          "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    FA_DBG_TMEM(taddr, 16u);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]),
          "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]),
          "=f"(v[14]), "=f"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    FA_DBG_TMEM(taddr, 32u);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
            taddr),
        "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]),
        "f"(v[8]), "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]),
        "f"(v[15]), "f"(v[16]), "f"(v[17]), "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]),
        "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]), "f"(v[27]), "f"(v[28]),
        "f"(v[29]), "f"(v[30]), "f"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    FA_DBG_TMEM(taddr, 16u);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15])
        : "memory");
}

// ----------------------------------------------------------------------------- CTA pairs (cta_group::2)
// A cluster of two CTAs on one TPC can run one MMA of M = 256: each CTA supplies the 128 rows of A that
// end up in its own tensor memory and half of B (N/2 columns), and one thread of the even-ranked CTA
// (the leader) issues the instruction for both.  The wrappers below are the pair forms of those above.
// Every CTA fetches its own tiles: no load is shared between CTAs.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// Arrival on an mbarrier of any CTA of the cluster (`bar` is a shared::cluster address).  What the arrival
// hands over here is tensor memory (scores read, P written, O read out), which the tcgen05 fences around the
// arrival and the wait order; the arrival itself carries the default semantics.  (Measured: with an explicit
// release at cluster scope on each of these arrivals the kernel took 1.6 times as many clocks.)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One arrival on the mbarrier at shared::cluster address `bar` (of either CTA of the pair) when every
// tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor of the pair form: M = 256 (128 rows in each CTA), fp16 A and B, fp32 D.
__host__ __device__ constexpr uint32_t make_idesc_f16_pair(uint32_t n, uint32_t b_mn_major) {
    return (1u << 4) | (b_mn_major << 16) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
// 3-D tiled load global -> this CTA's shared memory, completion (bytes) on an mbarrier that may belong
// to the other CTA of the pair (`bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* map, uint32_t bar, int32_t x, int32_t y,
                                                 int32_t z) {
    FA_DBG_COPY(dst, 4096u, x, y, z, false);
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ----------------------------------------------------------------------------- arithmetic
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two floats -> one 32-bit word of two fp16 values, `lo` in bits [0,16).
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Packed pairs of fp32 (one 64-bit register): two multiply-adds / adds per instruction.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Load with acquire semantics at device scope: loads that follow it in program order see what the
// writer of the value had made visible (with a release or a fence) before writing it.
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* ptr) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

// 32 bytes of read-only global memory with one instruction (the address must be 32-byte aligned)
__device__ __forceinline__ void ldg_256(const void* ptr, uint32_t (&w)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(ptr));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

}  // namespace fa
