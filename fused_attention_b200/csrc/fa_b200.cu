// C-ABI launcher of the sm_100a fused attention forward (declared in include/fa_b200.h).
// Torch-free: it needs the CUDA runtime only; the driver's cuTensorMapEncodeTiled is looked up at
// run time, so nothing links against libcuda.
//
// Replaces, in the reference: launch_attention_kernel<H, C> (include/fused_attn.cuh:860-894), the
// (head_dim, chunk_size) dispatch switch (src/fused_attn_extention.cu:72-111) and the
// print-and-exit error helpers (include/fused_attn.cuh:17-42).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <atomic>
#include <mutex>

#include "fa_b200.h"
#include "fa_kernels.cuh"
#include "fa_pair.cuh"

namespace {

using fa::Params;

constexpr int kMaxDevices = 64;
constexpr int kHostChunks = 8;   // pipeline depth of the host-buffer entry point
constexpr int kStatusWords = 4;  // device status block, see fa::WaitCtl

// bytes of one split-scratch buffer for a device with `sms` SMs: numerators, {max, sum} pairs, counters
size_t split_o_bytes(int sms) { return static_cast<size_t>(2 * sms) * 2 * (128 / 4) * fa::kTile * sizeof(float4); }
size_t split_ml_bytes(int sms) { return static_cast<size_t>(2 * sms) * 2 * fa::kTile * sizeof(float2); }
size_t split_cnt_bytes(int sms) { return static_cast<size_t>(sms) * 2 * 4 * sizeof(uint32_t); }

struct SplitScratch {
    bool taken = false;
    cudaStream_t stream = nullptr;
    float4* o = nullptr;       // fa::Params::part_o
    float2* ml = nullptr;      // fa::Params::part_ml
    uint32_t* cnt = nullptr;   // fa::Params::part_cnt
};
constexpr int kSplitPool = 4;

struct DeviceCtx {
    bool ready = false;
    int cc_major = 0, cc_minor = 0, sm_count = 0, smem_optin = 0;
    uint32_t* status = nullptr;   // device memory: {first failure code, reporting CTA count, id of the launch that reported, -}
    std::atomic<uint32_t> attr_done{0};   // bit per kernel instance whose smem attribute is set
    std::atomic<int> pair_clusters{-1};    // how many CTA pairs of fa_fwd_pair the device holds at once (-1: not asked yet)
    std::atomic<int> pair_clusters_mask{-1};   // the same for the instance with a mask
    // Scratch of launches that divide their last round of work items (fa::Plan): one buffer per stream,
    // because launches on different streams may run at the same time.  kSplitPool buffers are allocated
    // with the context; a launch on a stream that finds none free runs undivided.
    std::mutex split_mu;
    SplitScratch split[kSplitPool];
    // host-buffer entry point: copy-in / compute / copy-out streams, per-chunk events and
    // grow-on-demand staging buffers
    std::mutex host_mu;   // one host-buffer call at a time per device: they share the staging buffers
    cudaStream_t host_stream = nullptr, host_stream2 = nullptr, host_stream3 = nullptr;
    cudaEvent_t ev_in[8] = {}, ev_cmp[8] = {};
    void* stage[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};  // q k v y mask
    size_t stage_bytes[5] = {0, 0, 0, 0, 0};
};

DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mu;
std::atomic<uint32_t> g_launch_id{0};   // every launch gets its own non-zero id (Params::launch_id)

int fold_status(uint32_t* status_dev, uint32_t* const* counters, int n_counters, size_t counter_bytes);
int fold_ctx_status(DeviceCtx& c) {
    uint32_t* counters[kSplitPool];
    for (int i = 0; i < kSplitPool; ++i) counters[i] = c.split[i].cnt;
    return fold_status(c.status, counters, kSplitPool, split_cnt_bytes(c.sm_count));
}

uint32_t next_launch_id() {
    uint32_t id = g_launch_id.fetch_add(1, std::memory_order_relaxed) + 1u;
    if (id == 0) id = g_launch_id.fetch_add(1, std::memory_order_relaxed) + 1u;
    return id;
}

// Read the device status block after the stream has been synchronised; a report is cleared once it
// has been returned, so that it is given to one caller and later calls start clean.
// (A launch that gave up may have left the part counters of a divided round half counted: they are
// zeroed with the report.)
int fold_status(uint32_t* status_dev, uint32_t* const* counters, int n_counters, size_t counter_bytes) {
    uint32_t w[2] = {0, 0};
    cudaError_t e = cudaMemcpy(w, status_dev, sizeof(w), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (w[0] == 0) return FA_B200_OK;
    e = cudaMemset(status_dev, 0, 2 * sizeof(uint32_t));
    for (int i = 0; i < n_counters && e == cudaSuccess; ++i) e = cudaMemset(counters[i], 0, counter_bytes);
    return e != cudaSuccess ? static_cast<int>(e) : FA_B200_ERR_DEVICE_TIMEOUT;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

#ifdef FA_CYCLES
unsigned long long* g_cycles_buf = nullptr;  // device buffer of two clock values, set by fa_b200_debug_cycles
#endif


// Caller holds g_mu and has made `device` current.
int ensure_ctx(int device, DeviceCtx** out) {
    if (device < 0 || device >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
    DeviceCtx& c = g_ctx[device];
    if (!c.ready) {
        cudaDeviceProp prop;
        cudaError_t e = cudaGetDeviceProperties(&prop, device);
        if (e != cudaSuccess) return static_cast<int>(e);
        c.cc_major = prop.major;
        c.cc_minor = prop.minor;
        c.sm_count = prop.multiProcessorCount;
        c.smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
        e = cudaMalloc(reinterpret_cast<void**>(&c.status), kStatusWords * sizeof(uint32_t));
        if (e != cudaSuccess) return static_cast<int>(e);
        e = cudaMemset(c.status, 0, kStatusWords * sizeof(uint32_t));
        if (e != cudaSuccess) return static_cast<int>(e);
        for (int i = 0; i < kSplitPool; ++i) {
            char* base = nullptr;
            const size_t ob = split_o_bytes(c.sm_count), mb = split_ml_bytes(c.sm_count), cb = split_cnt_bytes(c.sm_count);
            e = cudaMalloc(reinterpret_cast<void**>(&base), ob + mb + cb);
            if (e != cudaSuccess) return static_cast<int>(e);
            c.split[i].o = reinterpret_cast<float4*>(base);
            c.split[i].ml = reinterpret_cast<float2*>(base + ob);
            c.split[i].cnt = reinterpret_cast<uint32_t*>(base + ob + mb);
            e = cudaMemset(c.split[i].cnt, 0, cb);
            if (e != cudaSuccess) return static_cast<int>(e);
        }
        c.ready = true;
    }
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
            (void)cudaGetLastError();
            return FA_B200_ERR_DRIVER;
        }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = &c;
    return FA_B200_OK;
}

// 3-D map {F, L, B} over a contiguous [B, L, F] fp16 array; box = 128 rows x min(H, 64) columns.
int make_map(CUtensorMap* map, const void* base, uint32_t B, uint32_t L, uint32_t F, uint32_t H,
             uint32_t box_rows = static_cast<uint32_t>(fa::kTile)) {
    const uint32_t box_cols = H < 64 ? H : 64;
    const cuuint64_t dims[3] = {F, L, B};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(F) * 2ull,
                                   static_cast<cuuint64_t>(F) * 2ull * L};
    const cuuint32_t box[3] = {box_cols, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle swz = box_cols == 64   ? CU_TENSOR_MAP_SWIZZLE_128B
                                   : box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                    : CU_TENSOR_MAP_SWIZZLE_32B;
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims,
                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FA_B200_OK : FA_B200_ERR_DRIVER;
}

// 3-D map {L keys, L rows, B} over a contiguous [B, L, L] fp16 mask; box = 128 rows x 64 keys.  Needs rows that
// start on 16-byte boundaries (L a multiple of 8, base aligned); the caller checks.
int make_mask_map(CUtensorMap* map, const void* base, uint32_t B, uint32_t L) {
    const cuuint64_t dims[3] = {L, L, B};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(L) * 2ull, static_cast<cuuint64_t>(L) * 2ull * L};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(fa::kTile), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FA_B200_OK : FA_B200_ERR_DRIVER;
}

bool is_pow2(uint32_t x) { return x != 0 && (x & (x - 1)) == 0; }

// Whether TMA can fetch tiles of the mask: every row of it starts on a 16-byte boundary.
bool mask_rows_aligned(const void* mask, uint32_t L) {
    return (L & 7u) == 0u && (reinterpret_cast<uintptr_t>(mask) & 15u) == 0u;
}

int validate(const void* q, const void* k, const void* v, const void* mask, const void* y, uint32_t B,
             uint32_t L, uint32_t F, uint32_t H, uint32_t chunk, uint32_t flags) {
    if (!q || !k || !v || !y) return FA_B200_ERR_NULL_POINTER;
    if (!(H == 16 || H == 32 || H == 64 || H == 128)) return FA_B200_ERR_HEAD_DIM;
    if (chunk != 0) {
        // the reference's rule set, src/fused_attn_extention.cu:46-47
        if (!is_pow2(chunk) || chunk < 16 || chunk > 128 || chunk > 2 * H) return FA_B200_ERR_CHUNK;
        if (chunk == 16 && H == 128) return FA_B200_ERR_CHUNK;
    }
    if (B == 0 || L == 0 || F == 0 || F % H != 0) return FA_B200_ERR_SHAPE;
    if (L > (1u << 30)) return FA_B200_ERR_SHAPE;
    // one CTA per query tile, head and batch entry on the x axis of the grid
    if (static_cast<uint64_t>((L + 127) / 128) * (F / H) * B > 0x7FFFFFFFull) return FA_B200_ERR_SHAPE;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(y);
    if (all & 15u) return FA_B200_ERR_ALIGNMENT;
    if (mask && (reinterpret_cast<uintptr_t>(mask) & 1u)) return FA_B200_ERR_ALIGNMENT;
    const uint32_t known = FA_B200_FLAG_FORCE_SIMPLE | FA_B200_FLAG_FORCE_PIPELINED | FA_B200_FLAG_SYNC |
                           FA_B200_FLAG_NO_OVERLAP | FA_B200_FLAG_NO_SPLIT | FA_B200_FLAG_FORCE_PAIR | FA_B200_FLAG_NO_PAIR;
    if (flags & ~known) return FA_B200_ERR_FLAGS;
    if (flags & FA_B200_FLAG_FORCE_PAIR) {
        if (H != 128 || (mask && !mask_rows_aligned(mask, L)) || (flags & (FA_B200_FLAG_FORCE_SIMPLE | FA_B200_FLAG_NO_PAIR)))
            return FA_B200_ERR_FLAGS;
    }
    if ((flags & FA_B200_FLAG_FORCE_SIMPLE) && (flags & FA_B200_FLAG_FORCE_PIPELINED)) return FA_B200_ERR_FLAGS;
    if ((flags & FA_B200_FLAG_FORCE_PIPELINED) && H < 64) return FA_B200_ERR_FLAGS;
    return FA_B200_OK;
}

// 1 = simple kernel, 2 = pipelined kernel.
int select_kernel(uint32_t B, uint32_t L, uint32_t F, uint32_t H, bool has_mask, uint32_t flags,
                  int sm_count) {
    if (flags & FA_B200_FLAG_FORCE_SIMPLE) return 1;
    if (flags & (FA_B200_FLAG_FORCE_PIPELINED | FA_B200_FLAG_FORCE_PAIR)) return 2;
    (void)has_mask;   // both kernels take the additive mask
    if (H < 64) return 1;
    // The pipelined kernel works on items of two query tiles (256 rows) on persistent CTAs.  It wins
    // as soon as there are enough items to occupy a good part of the SMs (measured: 39 vs 57 us on
    // B=64 R=16 L=197 H=64); a single partial tile or a handful of items goes to the simple kernel,
    // which has twice as many, smaller CTAs.
    // With few items the two are level up to about five key steps (7-14 us, mostly launch); from
    // there on the pipelined kernel wins however few items there are (measured: B=1 R=16 L=1024 H=128
    // 20.5 vs 24.6 us, B=1 R=4 L=2048 32.8 vs 41.9 us, B=1 R=2 L=4096 57 vs 79 us).
    const uint64_t pairs = static_cast<uint64_t>((L + 255) / 256) * (F / H) * B;
    if (L <= 128) return 1;
    if (L > 5 * 128) return 2;
    if (pairs * 2 < static_cast<uint64_t>(sm_count)) return 1;
    return 2;
}

// How the pipelined kernel's work items are spread over its CTAs (fa::Plan).
struct Schedule {
    uint32_t grid;         // CTAs
    uint32_t full_rounds;  // rounds of whole items
    uint32_t tail_items;   // items of the divided last round (0 = nothing divided)
    uint32_t tail_steps;   // tail_items * n
    uint32_t tail_grid;    // CTAs that share the tail key steps
};

// n_items work items of n key steps each on a device with `sms` SMs.  Undivided: min(sms, n_items) CTAs
// take whole items round-robin.  When the last round would leave most SMs idle, the key steps of its r
// items are dealt out evenly instead: each of the first tail_grid CTAs gets a contiguous range of them (at
// most two items touched) and the parts of an item are merged in the kernel.  tail_grid = min(sms, 2 r): a
// range is then at least half an item, so no item has more than three parts (what the kernel's merge is
// built for).  Dividing has a price, measured at about five key steps per CTA (one more segment boundary,
// the hand-over of a part through L2 and the merge, which reads 128 KB per other part of an item): it is
// done when what it saves beyond that is at least a twentieth of the CTA's work.
constexpr uint32_t kSplitCostSteps = 5;
Schedule make_schedule(uint32_t n_items, uint32_t n, uint32_t sms, bool allow_split) {
    Schedule s;
    s.grid = n_items < sms ? n_items : sms;
    s.full_rounds = (n_items + s.grid - 1) / s.grid;
    s.tail_items = 0;
    s.tail_steps = 0;
    s.tail_grid = 0;
    if (!allow_split || sms == 0 || n < 2) return s;
    const uint32_t r = n_items % sms;
    if (r == 0) return s;
    const uint32_t tg = 2u * r < sms ? 2u * r : sms;
    const uint64_t T = static_cast<uint64_t>(r) * n;
    if (T * tg > 0xFFFFFFFFull) return s;                 // the kernel's range arithmetic is 32-bit
    const uint32_t most = static_cast<uint32_t>((T + tg - 1) / tg);   // key steps of the busiest tail CTA
    const uint32_t least = static_cast<uint32_t>(T / tg);
    const uint64_t undivided = static_cast<uint64_t>(s.full_rounds) * n;          // key steps of the busiest CTA, whole items
    const uint64_t gain_needed = kSplitCostSteps + (undivided / 20 > 1 ? undivided / 20 : 1);
    if (static_cast<uint64_t>(most) + gain_needed >= n) return s;
    if (2u * least + 2u <= n) return s;                   // four parts would fit (cannot happen with tail_grid <= 2 r: guard)
    s.grid = n_items < sms ? tg : sms;
    s.full_rounds = n_items / sms;
    s.tail_items = r;
    s.tail_steps = static_cast<uint32_t>(T);
    s.tail_grid = tg;
    return s;
}

// Launch with or without the programmatic-stream-serialization attribute.  With it the kernel's
// CTAs may become resident while the previous kernel of the stream drains; the kernels wait for
// that kernel's completion (griddepcontrol.wait) before they touch global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t st,
                          bool overlap, const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int H, bool M>
int launch_simple(DeviceCtx& c, int slot, const CUtensorMap& mq, const CUtensorMap& mk,
                  const CUtensorMap& mv, const Params& p, cudaStream_t st, bool overlap) {
    constexpr int smem = 3 * fa::TileGeom<H>::kTileBytes + 1024;
    auto kern = fa::fa_fwd_simple<H, M>;
    if (!(c.attr_done.load(std::memory_order_acquire) & (1u << slot))) {   // setting it twice is harmless
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        c.attr_done.fetch_or(1u << slot, std::memory_order_release);
    }
    const dim3 grid(p.n_q_tiles * p.R * p.B, 1, 1);
    const cudaError_t e = launch_kernel(kern, grid, 128, smem, st, overlap, mq, mk, mv, p);
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

template <int H, bool M>
int launch_pipelined(DeviceCtx& c, int slot, const CUtensorMap& mq, const CUtensorMap& mk,
                     const CUtensorMap& mv, const CUtensorMap& my, const CUtensorMap& mm, const Params& p,
                     uint32_t n_ctas, cudaStream_t st, bool overlap) {
    constexpr int smem = fa::PipeCfg<H, M>::kSmemBytes;
    auto kern = fa::fa_fwd_pipelined<H, M>;
    if (!(c.attr_done.load(std::memory_order_acquire) & (1u << slot))) {   // setting it twice is harmless
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        c.attr_done.fetch_or(1u << slot, std::memory_order_release);
    }
    const dim3 grid(n_ctas, 1, 1);   // persistent: at most one CTA per SM
    const cudaError_t e = launch_kernel(kern, grid, 512, smem, st, overlap, mq, mk, mv, my, mm, p);
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// The split-scratch buffer of `st` on this device: the one it already has, else a free one, else none.
// None also while the stream is being captured.
const SplitScratch* scratch_for_stream(DeviceCtx& c, cudaStream_t st) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (cap != cudaStreamCaptureStatusNone) return nullptr;
    std::lock_guard<std::mutex> lk(c.split_mu);
    for (int i = 0; i < kSplitPool; ++i)
        if (c.split[i].taken && c.split[i].stream == st) return &c.split[i];
    for (int i = 0; i < kSplitPool; ++i)
        if (!c.split[i].taken) {
            c.split[i].taken = true;
            c.split[i].stream = st;
            return &c.split[i];
        }
    return nullptr;
}

// When the kernel on pairs of CTAs is taken: head_dim 128, a mask only if TMA can fetch its tiles (every row
// on a 16-byte boundary), whole work items (a call whose last
// round is divided stays on single CTAs), and a number of 256-row blocks per (batch, head) that is even or
// large, since a pair works on 512 rows and an odd block leaves one CTA of a pair without work.  Measured on
// the headline shape: the same SM clocks per launch as on single CTAs, but less shared-memory and L2 traffic,
// so under the power cap the SMs clock 2 to 3 % higher.  Without a mask it is left alone when the pairs of SMs
// get at most one work item each (`heads` = batch entries x heads): setting up and leaving in pairs then costs
// more than it gains (measured 1 to 1.5 % slower with one item per pair, equal with two, 2 % faster from three on);
// with a mask the pairs' mask buffer per query tile decides.
bool use_pair_kernel(uint32_t H, bool has_mask, bool mask_ok, uint32_t q_pairs, uint32_t heads, uint32_t sms,
                     uint32_t tail_steps, uint32_t flags) {
    if (H != 128 || (has_mask && !mask_ok) || (flags & FA_B200_FLAG_NO_PAIR)) return false;
    if (flags & FA_B200_FLAG_FORCE_PAIR) return true;
    if (tail_steps != 0) return false;
    if (!has_mask && static_cast<uint64_t>((q_pairs + 1u) / 2u) * heads <= sms / 2u) return false;
    return (q_pairs % 2u) == 0u || q_pairs >= 16u;
}

// The pair kernel: clusters of two CTAs, as many as the device holds at once (asked once per device).
template <bool kHasMask>
int launch_pair(DeviceCtx& c, const CUtensorMap& mq, const CUtensorMap& mkh, const CUtensorMap& mv,
                const CUtensorMap& my, const CUtensorMap& mm, const Params& p, uint32_t n_quad_items,
                cudaStream_t st, bool overlap, bool* launched) {
    constexpr int smem = fa::PairCfgT<kHasMask>::kSmemBytes;
    constexpr int slot = kHasMask ? 13 : 12;
    auto kern = fa::fa_fwd_pair<kHasMask>;
    *launched = false;
    if (!(c.attr_done.load(std::memory_order_acquire) & (1u << slot))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return static_cast<int>(e);
        c.attr_done.fetch_or(1u << slot, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(512, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    std::atomic<int>& held = kHasMask ? c.pair_clusters_mask : c.pair_clusters;
    int clusters = held.load(std::memory_order_acquire);
    if (clusters < 0) {
        cfg.gridDim = dim3(static_cast<unsigned>(c.sm_count) & ~1u, 1, 1);
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        if (n > c.sm_count / 2) n = c.sm_count / 2;
        held.store(n, std::memory_order_release);
        clusters = n;
    }
    if (clusters <= 0) return FA_B200_OK;   // the device cannot hold a pair: the caller takes the other kernel
    const uint32_t nc = n_quad_items < static_cast<uint32_t>(clusters) ? n_quad_items : static_cast<uint32_t>(clusters);
    cfg.gridDim = dim3(2 * nc, 1, 1);
    cfg.numAttrs = overlap ? 2u : 1u;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mq, mkh, mv, my, mm, p);
    *launched = true;
    return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// Device-pointer launch on `st`.  Caller holds no lock.
int forward_device(const void* q, const void* k, const void* v, const void* mask, void* y, uint32_t B,
                   uint32_t L, uint32_t F, uint32_t H, int device, cudaStream_t st, uint32_t flags) {
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    int rc = FA_B200_OK;
    DeviceCtx* c = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);   // only the once-per-device set-up is serialised
        rc = ensure_ctx(device, &c);
    }
    {
        if (rc == FA_B200_OK && c->cc_major != 10) rc = FA_B200_ERR_ARCH;
        if (rc == FA_B200_OK) {
            CUtensorMap mq, mk, mv;
            rc = make_map(&mq, q, B, L, F, H);
            if (rc == FA_B200_OK) rc = make_map(&mk, k, B, L, F, H);
            if (rc == FA_B200_OK) rc = make_map(&mv, v, B, L, F, H);
            if (rc == FA_B200_OK) {
                Params p;
                p.y = static_cast<__half*>(y);
                p.mask = static_cast<const __half*>(mask);
                p.status = c->status;
                p.B = B;
                p.L = L;
                p.F = F;
                p.launch_id = next_launch_id();
                p.n_kv_tiles = (L + fa::kTile - 1) / fa::kTile;
                p.n_q_tiles = p.n_kv_tiles;
                p.R = F / H;
                p.q_pairs = (L + 2 * fa::kTile - 1) / (2 * fa::kTile);
                p.n_items = p.q_pairs * p.R * B;
                p.scale_log2 = static_cast<float>(1.4426950408889634 / std::sqrt(static_cast<double>(H)));
                p.mask_to_score = static_cast<float>(std::sqrt(static_cast<double>(H)));
                p.mask_tma = 0;
#ifdef FA_CYCLES
                p.cycles = g_cycles_buf;
#endif
                p.full_rounds = p.tail_items = p.tail_steps = p.tail_grid = 0;
                p.part_slots = static_cast<uint32_t>(2 * c->sm_count);
#ifdef FA_DEBUG
                // checked build: rows the kernel fails to write stay NaN
                if ((e = cudaMemsetAsync(y, 0xFF, static_cast<size_t>(B) * L * F * sizeof(__half), st)) != cudaSuccess)
                    rc = static_cast<int>(e);
#endif
                p.part_o = nullptr;
                p.part_ml = nullptr;
                p.part_cnt = nullptr;
                const int which = select_kernel(B, L, F, H, mask != nullptr, flags, c->sm_count);
                const bool overlap = (flags & FA_B200_FLAG_NO_OVERLAP) == 0;
                if (which == 2) {
                    // Dividing the last round needs scratch that no other launch is using: the buffer that
                    // belongs to this stream.  A stream that is being captured gets none (the recorded launch
                    // could later be replayed next to anything).
                    const SplitScratch* scratch = nullptr;
                    if (!(flags & (FA_B200_FLAG_NO_SPLIT | FA_B200_FLAG_FORCE_PAIR))) scratch = scratch_for_stream(*c, st);
                    const Schedule sch = make_schedule(p.n_items, p.n_kv_tiles, static_cast<uint32_t>(c->sm_count),
                                                       scratch != nullptr);
                    p.full_rounds = sch.full_rounds;
                    p.tail_items = sch.tail_items;
                    p.tail_steps = sch.tail_steps;
                    p.tail_grid = sch.tail_grid;
                    if (sch.tail_steps != 0) {
                        p.part_o = scratch->o;
                        p.part_ml = scratch->ml;
                        p.part_cnt = scratch->cnt;
                    }
                    // Y as a TMA store target: boxes of 32 rows x 64 columns (one epilogue warp each)
                    CUtensorMap my;
                    rc = make_map(&my, y, B, L, F, H, 32);
                    bool done = false;
                    // mask tiles through TMA when every mask row starts on a 16-byte boundary; else the
                    // softmax threads (of the kernel on single CTAs) read their rows straight from global memory
                    CUtensorMap mm = mq;
                    p.mask_tma = (mask && mask_rows_aligned(mask, L)) ? 1u : 0u;
                    if (rc == FA_B200_OK && p.mask_tma) rc = make_mask_map(&mm, mask, B, L);
                    if (rc == FA_B200_OK && use_pair_kernel(H, mask != nullptr, p.mask_tma != 0u, p.q_pairs, p.R * B,
                                                            static_cast<uint32_t>(c->sm_count), sch.tail_steps, flags)) {
                        // K as halves of a tile: boxes of 64 keys x 64 columns
                        CUtensorMap mkh;
                        rc = make_map(&mkh, k, B, L, F, H, 64);
                        if (rc == FA_B200_OK) {
                            Params pp = p;
                            pp.full_rounds = pp.tail_items = pp.tail_steps = pp.tail_grid = 0;
                            const uint32_t quads = ((p.q_pairs + 1u) / 2u) * p.R * B;
                            rc = mask ? launch_pair<true>(*c, mq, mkh, mv, my, mm, pp, quads, st, overlap, &done)
                                      : launch_pair<false>(*c, mq, mkh, mv, my, mm, pp, quads, st, overlap, &done);
                        }
                    }
                    if (rc == FA_B200_OK && !done) {
                        if (mask) {
                            if (rc == FA_B200_OK)
                                rc = H == 128 ? launch_pipelined<128, true>(*c, 10, mq, mk, mv, my, mm, p, sch.grid, st, overlap)
                                              : launch_pipelined<64, true>(*c, 11, mq, mk, mv, my, mm, p, sch.grid, st, overlap);
                        } else {
                            rc = H == 128 ? launch_pipelined<128, false>(*c, 8, mq, mk, mv, my, mq, p, sch.grid, st, overlap)
                                          : launch_pipelined<64, false>(*c, 9, mq, mk, mv, my, mq, p, sch.grid, st, overlap);
                        }
                    }
                } else if (mask) {
                    switch (H) {
                        case 16: rc = launch_simple<16, true>(*c, 4, mq, mk, mv, p, st, overlap); break;
                        case 32: rc = launch_simple<32, true>(*c, 5, mq, mk, mv, p, st, overlap); break;
                        case 64: rc = launch_simple<64, true>(*c, 6, mq, mk, mv, p, st, overlap); break;
                        default: rc = launch_simple<128, true>(*c, 7, mq, mk, mv, p, st, overlap); break;
                    }
                } else {
                    switch (H) {
                        case 16: rc = launch_simple<16, false>(*c, 0, mq, mk, mv, p, st, overlap); break;
                        case 32: rc = launch_simple<32, false>(*c, 1, mq, mk, mv, p, st, overlap); break;
                        case 64: rc = launch_simple<64, false>(*c, 2, mq, mk, mv, p, st, overlap); break;
                        default: rc = launch_simple<128, false>(*c, 3, mq, mk, mv, p, st, overlap); break;
                    }
                }
            }
        }
    }
    if (rc == FA_B200_OK && (flags & FA_B200_FLAG_SYNC)) {
        e = cudaStreamSynchronize(st);
        rc = e != cudaSuccess ? static_cast<int>(e) : fold_ctx_status(*c);
    }
    if (prev != device) (void)cudaSetDevice(prev);
    return rc;
}

int grow(DeviceCtx& c, int i, size_t bytes) {
    if (c.stage_bytes[i] >= bytes) return FA_B200_OK;
    if (c.stage[i]) (void)cudaFree(c.stage[i]);
    c.stage[i] = nullptr;
    c.stage_bytes[i] = 0;
    cudaError_t e = cudaMalloc(&c.stage[i], bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    c.stage_bytes[i] = bytes;
    return FA_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Scratch of the no-allocation entry point: one status pair {failure code, count} per CTA of the
// one-tile-per-CTA kernel.  File-scope device memory: every GPU that loads this library holds these
// 128 KiB until the process exits.  In host code the name `g_noalloc_status` is only a handle for
// cudaGetSymbolAddress; the kernel must be given the address that call returns.
constexpr uint32_t kNoAllocMaxCtas = 16384;
static __device__ __align__(256) uint32_t g_noalloc_status[2 * kNoAllocMaxCtas];

struct NoAllocCtx {
    std::mutex mu;                   // set-up and the attribute bits of this device
    bool ready = false;
    uint32_t* status_dev = nullptr;  // device address of g_noalloc_status on this device
    uint32_t attr_done = 0;
};
NoAllocCtx g_noalloc[kMaxDevices];

template <int H, bool M>
int launch_simple_noalloc(NoAllocCtx& c, int slot, const CUtensorMap& mq, const CUtensorMap& mk,
                          const CUtensorMap& mv, const Params& p, dim3 grid, cudaStream_t st) {
    constexpr int smem = 3 * fa::TileGeom<H>::kTileBytes + 1024;
    auto kern = fa::fa_fwd_simple<H, M, true>;
    {
        std::lock_guard<std::mutex> lk(c.mu);
        if (!(c.attr_done & (1u << slot))) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return static_cast<int>(e);
            c.attr_done |= (1u << slot);
        }
    }
    kern<<<grid, 128, smem, st>>>(mq, mk, mv, p);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" {

int fa_b200_attention_forward_noalloc(const void* q, const void* k, const void* v, const void* mask_or_null,
                                      void* y, uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                                      uint32_t chunk_hint, int device, void* cuda_stream, uint32_t flags) {
    if (flags & ~static_cast<uint32_t>(FA_B200_FLAG_SYNC)) return FA_B200_ERR_FLAGS;  // one kernel: nothing to force
    int rc = validate(q, k, v, mask_or_null, y, B, L, F, head_dim, chunk_hint, flags);
    if (rc != FA_B200_OK) return rc;
    const uint32_t H = head_dim;
    const uint32_t n_q_tiles = (L + fa::kTile - 1) / fa::kTile;
    const uint64_t ctas = static_cast<uint64_t>(n_q_tiles) * (F / H) * B;
    if (ctas > kNoAllocMaxCtas) return FA_B200_ERR_TOO_LARGE;
    if (device < 0 || device >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
    const dim3 grid(static_cast<uint32_t>(ctas), 1, 1);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);

    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return static_cast<int>(e);
    NoAllocCtx& c = g_noalloc[device];
    {
        // Set-up, once per device, with that device current: the compute capability is checked first
        // (the scratch array only exists in the sm_100a image), then the device address of the
        // file-scope scratch is looked up.  No allocation.  Calls on other devices do not wait here.
        std::lock_guard<std::mutex> lk(c.mu);
        if (!c.ready) {
            int major = 0;
            e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
            if (e != cudaSuccess) {
                rc = static_cast<int>(e);
            } else if (major != 10) {
                rc = FA_B200_ERR_ARCH;
            } else {
                void* sym = nullptr;
                e = cudaGetSymbolAddress(&sym, g_noalloc_status);
                if (e != cudaSuccess) {
                    rc = static_cast<int>(e);
                } else {
                    c.status_dev = static_cast<uint32_t*>(sym);
                    c.ready = true;
                }
            }
        }
    }
    if (rc == FA_B200_OK) {
        std::lock_guard<std::mutex> lk(g_mu);   // the driver's tensor-map encoder is looked up once per process
        if (g_encode == nullptr) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
                (void)cudaGetLastError();
                rc = FA_B200_ERR_DRIVER;
            } else {
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            }
        }
    }
    CUtensorMap mq, mk, mv;
    if (rc == FA_B200_OK) rc = make_map(&mq, q, B, L, F, H);
    if (rc == FA_B200_OK) rc = make_map(&mk, k, B, L, F, H);
    if (rc == FA_B200_OK) rc = make_map(&mv, v, B, L, F, H);
    if (rc == FA_B200_OK) {
        // The array keeps what the previous call left: zero the pairs this grid will use, in
        // stream order ahead of the kernel.
        e = cudaMemsetAsync(c.status_dev, 0, static_cast<size_t>(ctas) * 2 * sizeof(uint32_t), st);
        if (e != cudaSuccess) rc = static_cast<int>(e);
    }
    if (rc == FA_B200_OK) {
        Params p;
        p.y = static_cast<__half*>(y);
        p.mask = static_cast<const __half*>(mask_or_null);
        p.status = c.status_dev;   // the address from cudaGetSymbolAddress, never the symbol itself
        p.launch_id = 0;           // per-CTA status pairs: no launch word
        p.B = B;
        p.L = L;
        p.F = F;
        p.n_kv_tiles = n_q_tiles;
        p.n_q_tiles = n_q_tiles;
        p.R = F / H;
        p.q_pairs = (L + 2 * fa::kTile - 1) / (2 * fa::kTile);
        p.n_items = p.q_pairs * p.R * B;
        p.scale_log2 = static_cast<float>(1.4426950408889634 / std::sqrt(static_cast<double>(H)));
        p.mask_to_score = static_cast<float>(std::sqrt(static_cast<double>(H)));
        p.mask_tma = 0;
        p.full_rounds = p.tail_items = p.tail_steps = p.tail_grid = 0;
        p.part_slots = 0;
        p.part_o = nullptr;
        p.part_ml = nullptr;
        p.part_cnt = nullptr;
#ifdef FA_CYCLES
        p.cycles = nullptr;
#endif
        if (mask_or_null) {
            switch (H) {
                case 16: rc = launch_simple_noalloc<16, true>(c, 4, mq, mk, mv, p, grid, st); break;
                case 32: rc = launch_simple_noalloc<32, true>(c, 5, mq, mk, mv, p, grid, st); break;
                case 64: rc = launch_simple_noalloc<64, true>(c, 6, mq, mk, mv, p, grid, st); break;
                default: rc = launch_simple_noalloc<128, true>(c, 7, mq, mk, mv, p, grid, st); break;
            }
        } else {
            switch (H) {
                case 16: rc = launch_simple_noalloc<16, false>(c, 0, mq, mk, mv, p, grid, st); break;
                case 32: rc = launch_simple_noalloc<32, false>(c, 1, mq, mk, mv, p, grid, st); break;
                case 64: rc = launch_simple_noalloc<64, false>(c, 2, mq, mk, mv, p, grid, st); break;
                default: rc = launch_simple_noalloc<128, false>(c, 3, mq, mk, mv, p, grid, st); break;
            }
        }
    }
    if (rc == FA_B200_OK && (flags & FA_B200_FLAG_SYNC)) {
        e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = static_cast<int>(e);
        // read the status pairs back through a fixed buffer on the stack
        uint32_t buf[512];
        for (uint64_t off = 0; rc == FA_B200_OK && off < ctas * 2; off += 512) {
            const size_t cnt = static_cast<size_t>(ctas * 2 - off < 512 ? ctas * 2 - off : 512);
            e = cudaMemcpy(buf, c.status_dev + off, cnt * sizeof(uint32_t), cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) { rc = static_cast<int>(e); break; }
            for (size_t i = 0; i < cnt; i += 2)
                if (buf[i] != 0) { rc = FA_B200_ERR_DEVICE_TIMEOUT; break; }
        }
    }
    if (prev != device) (void)cudaSetDevice(prev);
    return rc;
}

int fa_b200_attention_forward(const void* q, const void* k, const void* v, const void* mask_or_null,
                              void* y, uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                              uint32_t chunk_hint, int device, void* cuda_stream, uint32_t flags) {
    const int rc = validate(q, k, v, mask_or_null, y, B, L, F, head_dim, chunk_hint, flags);
    if (rc != FA_B200_OK) return rc;
    return forward_device(q, k, v, mask_or_null, y, B, L, F, head_dim, device,
                          static_cast<cudaStream_t>(cuda_stream), flags);
}

int fa_b200_attention_forward_host(const void* q, const void* k, const void* v, const void* mask_or_null,
                                   void* y, uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                                   uint32_t chunk_hint, int device, uint32_t flags) {
    // Host pointers need no 16-byte alignment; validate everything else with aligned stand-ins.
    if (!q || !k || !v || !y) return FA_B200_ERR_NULL_POINTER;
    alignas(16) static const char aligned_dummy[16] = {0};
    int rc = validate(aligned_dummy, aligned_dummy, aligned_dummy, mask_or_null ? aligned_dummy : nullptr,
                      aligned_dummy, B, L, F, head_dim, chunk_hint, flags);
    if (rc != FA_B200_OK) return rc;
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    const size_t bytes = static_cast<size_t>(B) * L * F * sizeof(__half);
    const size_t mbytes = mask_or_null ? static_cast<size_t>(B) * L * L * sizeof(__half) : 0;
    DeviceCtx* c = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        rc = ensure_ctx(device, &c);
        if (rc == FA_B200_OK && c->host_stream == nullptr) {
            e = cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->host_stream2, cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->host_stream3, cudaStreamNonBlocking);
            for (int i = 0; i < kHostChunks && e == cudaSuccess; ++i) {
                e = cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming);
                if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_cmp[i], cudaEventDisableTiming);
            }
            if (e != cudaSuccess) rc = static_cast<int>(e);
        }
    }
    std::unique_lock<std::mutex> host_lock;
    if (rc == FA_B200_OK) host_lock = std::unique_lock<std::mutex>(c->host_mu);
    if (rc == FA_B200_OK) {
        // the staging buffers are sized under the device's host lock, so a concurrent call cannot
        // free them while this one is using them
        for (int i = 0; i < 4 && rc == FA_B200_OK; ++i) rc = grow(*c, i, bytes);
        if (rc == FA_B200_OK && mbytes) rc = grow(*c, 4, mbytes);
    }
    if (rc == FA_B200_OK) {
        // Chunked pipeline over three streams: while chunk c computes, chunk c+1 is copied in and
        // chunk c-1 is copied out (PCIe carries both directions at once).  Chunks are groups of
        // batch entries (contiguous in host memory) when B >= 2, otherwise groups of heads moved
        // with pitched copies into compact [B, L, heads*H] device slices.
        cudaStream_t s_in = c->host_stream, s_cmp = c->host_stream2, s_out = c->host_stream3;
        const uint32_t H = head_dim, R = F / H;
        const bool by_batch = B >= 2;
        const uint32_t units = by_batch ? B : R;
        const uint32_t n_chunks = units < kHostChunks ? units : kHostChunks;
        const __half* hsrc[3] = {static_cast<const __half*>(q), static_cast<const __half*>(k),
                                 static_cast<const __half*>(v)};
        // every chunk runs the kernel the whole problem would get, with every work item undivided, so
        // the result has the same bits as one device-pointer call on the full tensors with
        // FA_B200_FLAG_NO_SPLIT
        // (plain launches: a chunk's kernel is ordered behind copies on other streams, not behind a kernel)
        const uint32_t chunk_flags =
            (flags & ~static_cast<uint32_t>(FA_B200_FLAG_SYNC | FA_B200_FLAG_FORCE_SIMPLE | FA_B200_FLAG_FORCE_PIPELINED)) |
            FA_B200_FLAG_NO_OVERLAP | FA_B200_FLAG_NO_SPLIT |
            (select_kernel(B, L, F, H, mask_or_null != nullptr, flags, c->sm_count) == 2 ? FA_B200_FLAG_FORCE_PIPELINED
                                                                                       : FA_B200_FLAG_FORCE_SIMPLE);
        if (mbytes && !by_batch) {   // the mask is shared by all heads: one copy ahead of everything
            e = cudaMemcpyAsync(c->stage[4], mask_or_null, mbytes, cudaMemcpyHostToDevice, s_in);
            if (e != cudaSuccess) rc = static_cast<int>(e);
        }
        size_t dev_off = 0;   // elements into the staging buffers
        for (uint32_t ch = 0; ch < n_chunks && rc == FA_B200_OK; ++ch) {
            const uint32_t u0 = static_cast<uint32_t>(static_cast<uint64_t>(units) * ch / n_chunks);
            const uint32_t u1 = static_cast<uint32_t>(static_cast<uint64_t>(units) * (ch + 1) / n_chunks);
            const uint32_t nu = u1 - u0;
            if (nu == 0) continue;
            const uint32_t cB = by_batch ? nu : B, cF = by_batch ? F : nu * H;
            const size_t elems = static_cast<size_t>(cB) * L * cF;
            __half* d[4];
            for (int i = 0; i < 4; ++i) d[i] = static_cast<__half*>(c->stage[i]) + dev_off;
            const __half* dmask = nullptr;
            for (int i = 0; i < 3 && rc == FA_B200_OK; ++i) {
                if (by_batch)
                    e = cudaMemcpyAsync(d[i], hsrc[i] + static_cast<size_t>(u0) * L * F, elems * sizeof(__half),
                                        cudaMemcpyHostToDevice, s_in);
                else
                    e = cudaMemcpy2DAsync(d[i], static_cast<size_t>(cF) * sizeof(__half), hsrc[i] + static_cast<size_t>(u0) * H,
                                          static_cast<size_t>(F) * sizeof(__half), static_cast<size_t>(cF) * sizeof(__half),
                                          static_cast<size_t>(B) * L, cudaMemcpyHostToDevice, s_in);
                if (e != cudaSuccess) rc = static_cast<int>(e);
            }
            if (rc == FA_B200_OK && mbytes) {
                if (by_batch) {
                    const size_t moff = static_cast<size_t>(u0) * L * L;
                    e = cudaMemcpyAsync(static_cast<__half*>(c->stage[4]) + moff,
                                        static_cast<const __half*>(mask_or_null) + moff,
                                        static_cast<size_t>(nu) * L * L * sizeof(__half), cudaMemcpyHostToDevice, s_in);
                    if (e != cudaSuccess) rc = static_cast<int>(e);
                    dmask = static_cast<const __half*>(c->stage[4]) + moff;
                } else {
                    dmask = static_cast<const __half*>(c->stage[4]);
                }
            }
            if (rc == FA_B200_OK && (e = cudaEventRecord(c->ev_in[ch], s_in)) != cudaSuccess) rc = static_cast<int>(e);
            if (rc == FA_B200_OK && (e = cudaStreamWaitEvent(s_cmp, c->ev_in[ch], 0)) != cudaSuccess) rc = static_cast<int>(e);
            if (rc == FA_B200_OK)
                rc = forward_device(d[0], d[1], d[2], dmask, d[3], cB, L, cF, head_dim, device, s_cmp, chunk_flags);
            if (rc == FA_B200_OK && (e = cudaEventRecord(c->ev_cmp[ch], s_cmp)) != cudaSuccess) rc = static_cast<int>(e);
            if (rc == FA_B200_OK && (e = cudaStreamWaitEvent(s_out, c->ev_cmp[ch], 0)) != cudaSuccess) rc = static_cast<int>(e);
            if (rc == FA_B200_OK) {
                __half* hy = static_cast<__half*>(y);
                if (by_batch)
                    e = cudaMemcpyAsync(hy + static_cast<size_t>(u0) * L * F, d[3], elems * sizeof(__half),
                                        cudaMemcpyDeviceToHost, s_out);
                else
                    e = cudaMemcpy2DAsync(hy + static_cast<size_t>(u0) * H, static_cast<size_t>(F) * sizeof(__half), d[3],
                                          static_cast<size_t>(cF) * sizeof(__half), static_cast<size_t>(cF) * sizeof(__half),
                                          static_cast<size_t>(B) * L, cudaMemcpyDeviceToHost, s_out);
                if (e != cudaSuccess) rc = static_cast<int>(e);
            }
            dev_off += elems;
        }
        // all three streams drain before the staging buffers may be reused or the result read
        cudaError_t e1 = cudaStreamSynchronize(s_in), e2 = cudaStreamSynchronize(s_cmp), e3 = cudaStreamSynchronize(s_out);
        if (rc == FA_B200_OK && e1 != cudaSuccess) rc = static_cast<int>(e1);
        if (rc == FA_B200_OK && e2 != cudaSuccess) rc = static_cast<int>(e2);
        if (rc == FA_B200_OK && e3 != cudaSuccess) rc = static_cast<int>(e3);
        if (rc == FA_B200_OK) rc = fold_ctx_status(*c);
    }
    if (prev != device) (void)cudaSetDevice(prev);
    return rc;
}

const char* fa_b200_strerror(int code) {
    switch (code) {
        case FA_B200_OK: return "success";
        case FA_B200_ERR_NULL_POINTER: return "q, k, v and y must not be NULL";
        case FA_B200_ERR_HEAD_DIM: return "head_dim must be 16, 32, 64 or 128";
        case FA_B200_ERR_CHUNK:
            return "chunk_size must be a power of two in [16, 128], at most 2*head_dim, and not 16 with head_dim 128";
        case FA_B200_ERR_SHAPE: return "B, L, F must be positive, F divisible by head_dim, and ceil(L/128)*(F/head_dim)*B below 2^31";
        case FA_B200_ERR_ALIGNMENT: return "q, k, v and y must be 16-byte aligned";
        case FA_B200_ERR_ARCH: return "the device is not compute capability 10.x (sm_100a)";
        case FA_B200_ERR_DRIVER: return "cuTensorMapEncodeTiled is unavailable or rejected the tensor";
        case FA_B200_ERR_FLAGS: return "unknown or contradictory flags";
        case FA_B200_ERR_DEVICE_TIMEOUT: return "a bounded wait inside the kernel expired; see fa_b200_read_status";
        case FA_B200_ERR_TOO_LARGE: return "the problem exceeds the fixed capacity of this entry point";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown fa_b200 status";
}

int fa_b200_query(int device, int32_t out[4]) {
    if (!out) return FA_B200_ERR_NULL_POINTER;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return static_cast<int>(e);
    out[0] = prop.major;
    out[1] = prop.minor;
    out[2] = prop.multiProcessorCount;
    out[3] = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
    return FA_B200_OK;
}

int fa_b200_read_status(int device, uint32_t out[2]) {
    if (!out) return FA_B200_ERR_NULL_POINTER;
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return static_cast<int>(e);
    int rc = FA_B200_OK;
    DeviceCtx* c = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        rc = ensure_ctx(device, &c);
    }
    if (rc == FA_B200_OK) {
        e = cudaDeviceSynchronize();
        if (e == cudaSuccess) e = cudaMemcpy(out, c->status, 2 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemset(c->status, 0, kStatusWords * sizeof(uint32_t));
        if (e == cudaSuccess && (out[0] != 0 || out[1] != 0))
            for (int i = 0; i < kSplitPool && e == cudaSuccess; ++i)
                e = cudaMemset(c->split[i].cnt, 0, split_cnt_bytes(c->sm_count));
        if (e != cudaSuccess) rc = static_cast<int>(e);
    }
    if (prev != device) (void)cudaSetDevice(prev);
    return rc;
}

int fa_b200_selftest_bounded_wait(int device, uint32_t out[3]) {
    if (!out) return FA_B200_ERR_NULL_POINTER;
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return static_cast<int>(e);
    int rc = FA_B200_OK;
    uint32_t* scratch = nullptr;  // {status code, reporting CTAs, returned marker}
    e = cudaMalloc(reinterpret_cast<void**>(&scratch), 3 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(scratch, 0, 3 * sizeof(uint32_t));
    if (e == cudaSuccess) {
        // 20 million cycles: about 10 ms
        fa::fa_selftest_bounded_wait<<<1, 32>>>(scratch, fa::kRoleDrain | 0x7Fu, 20000000LL, scratch + 2);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(out, scratch, 3 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (scratch) (void)cudaFree(scratch);
    if (e != cudaSuccess) rc = static_cast<int>(e);
    if (prev != device) (void)cudaSetDevice(prev);
    return rc;
}

int fa_b200_selftest_debug_checks(int device, uint32_t out[4]) {
    if (!out) return FA_B200_ERR_NULL_POINTER;
    out[0] = out[1] = out[2] = out[3] = 0;
#ifdef FA_DEBUG
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (prev != device && (e = cudaSetDevice(device)) != cudaSuccess) return static_cast<int>(e);
    uint32_t* scratch = nullptr;   // {status code, reporting CTAs, launch word, bit mask of the predicates' answers}
    e = cudaMalloc(reinterpret_cast<void**>(&scratch), 4 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(scratch, 0, 4 * sizeof(uint32_t));
    if (e == cudaSuccess) {
        fa::fa_selftest_debug_checks<<<1, 32>>>(scratch);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(out, scratch, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (scratch) (void)cudaFree(scratch);
    out[2] = 1;   // this is a checked build
    if (prev != device) (void)cudaSetDevice(prev);
    return e != cudaSuccess ? static_cast<int>(e) : FA_B200_OK;
#else
    (void)device;
    return FA_B200_OK;
#endif
}

#ifdef FA_CYCLES
// -DFA_CYCLES builds only: CTA 0 of the pipelined kernel writes its time stamps here (64 records of 4 u64).
int fa_b200_debug_cycles(void* device_buffer_of_256_u64) {
    g_cycles_buf = static_cast<unsigned long long*>(device_buffer_of_256_u64);
    return FA_B200_OK;
}
#endif

int fa_b200_describe_schedule(uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim, uint32_t flags,
                              uint32_t sm_count, uint32_t out[7]) {
    if (!out) return FA_B200_ERR_NULL_POINTER;
    alignas(16) static const char d[16] = {0};
    const int rc = validate(d, d, d, nullptr, d, B, L, F, head_dim, 0, flags);
    if (rc != FA_B200_OK) return rc;
    const uint32_t n = (L + fa::kTile - 1) / fa::kTile;
    const uint32_t n_items = ((L + 2 * fa::kTile - 1) / (2 * fa::kTile)) * (F / head_dim) * B;
    const int which = select_kernel(B, L, F, head_dim, false, flags, static_cast<int>(sm_count));
    out[0] = static_cast<uint32_t>(which);
    out[5] = n;
    if (which != 2) {
        out[1] = n * (F / head_dim) * B;
        out[2] = out[3] = out[4] = out[6] = 0;
        return FA_B200_OK;
    }
    const Schedule s = make_schedule(n_items, n, sm_count,
                                     (flags & (FA_B200_FLAG_NO_SPLIT | FA_B200_FLAG_FORCE_PAIR)) == 0);
    const uint32_t q_pairs = (L + 2 * fa::kTile - 1) / (2 * fa::kTile);
    if (use_pair_kernel(head_dim, false, true, q_pairs, (F / head_dim) * B, sm_count, s.tail_steps, flags) && sm_count >= 2) {
        // pairs of CTAs: work items of 512 query rows, one cluster of two CTAs per pair of SMs
        const uint32_t quads = ((q_pairs + 1) / 2) * (F / head_dim) * B, clusters = quads < sm_count / 2 ? quads : sm_count / 2;
        out[0] = 3;
        out[1] = 2 * clusters;
        out[2] = (quads + clusters - 1) / clusters;
        out[3] = out[4] = out[6] = 0;
        return FA_B200_OK;
    }
    out[1] = s.grid;
    out[2] = s.full_rounds;
    out[3] = s.tail_items;
    out[4] = s.tail_steps;
    out[6] = s.tail_grid;
    return FA_B200_OK;
}

int fa_b200_select_kernel(uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim, int has_mask,
                          uint32_t flags) {
    alignas(16) static const char d[16] = {0};
    const int rc = validate(d, d, d, has_mask ? d : nullptr, d, B, L, F, head_dim, 0, flags);
    if (rc != FA_B200_OK) return rc;
    // the SM count of the current device decides, as it does in a launch; 148 (B200) without a device
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        sms = 148;
    }
    const int which = select_kernel(B, L, F, head_dim, has_mask != 0, flags, sms);
    if (which != 2) return which;
    const uint32_t n = (L + fa::kTile - 1) / fa::kTile, q_pairs = (L + 2 * fa::kTile - 1) / (2 * fa::kTile);
    const Schedule s = make_schedule(q_pairs * (F / head_dim) * B, n, static_cast<uint32_t>(sms),
                                     (flags & (FA_B200_FLAG_NO_SPLIT | FA_B200_FLAG_FORCE_PAIR)) == 0);
    // (a mask is taken to start on a 16-byte boundary here)
    return use_pair_kernel(head_dim, has_mask != 0, (L & 7u) == 0u, q_pairs, (F / head_dim) * B,
                           static_cast<uint32_t>(sms), s.tail_steps, flags) ? 3 : 2;
}

}  // extern "C"
