/*
 * fa_b200.h — C ABI of the B200 (sm_100a) fused multi-head attention forward.
 *
 * One operator:  Y = softmax(Q K^T / sqrt(H)) V  per (batch, head), fp16 in / fp16 out,
 * fp32 accumulation and fp32 online-softmax state, no L x L score matrix in global memory.
 *
 * Tensor contract (same as the reference operator, src/fused_attn_extention.cu:24-70):
 * q, k, v, y are contiguous fp16 device arrays of logical shape [B, L, F] with F = R * head_dim
 * (any B, R, L with ceil(L/128) * R * B below 2^31);
 * head h owns columns [h*head_dim, (h+1)*head_dim) of the last axis
 * (include/fused_attn.cuh:681-696 in the reference).  The optional mask is a contiguous fp16
 * array [B, L, L] that is ADDED to the scaled scores of every head (reference
 * include/fused_attn.cuh:686,735-742; the reference adds it to the first key chunk only, this
 * library adds it to every key tile).
 *
 * Every function is thread-safe.  None of them terminates the process: where the reference
 * launcher prints and calls exit() (include/fused_attn.cuh:17-42) these return a status code.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  0 = success, negative = rejected before launch, positive = a cudaError_t. */
enum {
    FA_B200_OK = 0,
    FA_B200_ERR_NULL_POINTER = -1,   /* q, k, v or y is NULL                                   */
    FA_B200_ERR_HEAD_DIM = -2,       /* head_dim not in {16, 32, 64, 128}                      */
    FA_B200_ERR_CHUNK = -3,          /* chunk_hint violates the reference's rule set           */
    FA_B200_ERR_SHAPE = -4,          /* B, L or F is zero, F % head_dim != 0, or too large     */
    FA_B200_ERR_ALIGNMENT = -5,      /* a tensor base address is not 16-byte aligned           */
    FA_B200_ERR_ARCH = -6,           /* the device is not compute capability 10.x              */
    FA_B200_ERR_DRIVER = -7,         /* cuTensorMapEncodeTiled unavailable or failed           */
    FA_B200_ERR_FLAGS = -8,          /* contradictory or unknown flag bits                     */
    FA_B200_ERR_DEVICE_TIMEOUT = -9, /* a bounded device-side wait expired (see read_status)   */
    FA_B200_ERR_TOO_LARGE = -10      /* a fixed-capacity entry point was given too much work   */
};

/* flags for fa_b200_attention_forward */
enum {
    FA_B200_FLAG_DEFAULT = 0u,
    FA_B200_FLAG_FORCE_SIMPLE = 1u,    /* always use the one-tile-per-CTA kernel                */
    FA_B200_FLAG_FORCE_PIPELINED = 2u, /* always use the warp-specialised kernel (H in {64,128}) */
    FA_B200_FLAG_SYNC = 4u,            /* synchronise the stream before returning and fold the
                                          device status word into the return value; a report is
                                          cleared when it is returned (see fa_b200_read_status) */
    FA_B200_FLAG_NO_OVERLAP = 8u,      /* plain launch.  By default the kernel is launched with the
                                          programmatic-stream-serialization attribute: its CTAs may
                                          become resident and set up their barriers and tensor memory
                                          while the previous kernel of the stream drains; they touch
                                          global memory only once that kernel has completed, so the
                                          stream's ordering guarantees are unchanged             */
    FA_B200_FLAG_FORCE_PAIR = 32u,     /* head_dim 128 (with a mask: one whose rows all start on 16-byte
                                          boundaries, else FA_B200_ERR_FLAGS): always use the kernel
                                          that runs on pairs
                                          of CTAs (one MMA of 256 rows for two SMs); implies whole work
                                          items.  By default it is taken for such calls when their last
                                          round is not divided, the sequence has an even or large
                                          number of 256-row blocks and (without a mask) the pairs of SMs
                                          get more than one work item each                           */
    FA_B200_FLAG_NO_PAIR = 64u,        /* never use that kernel                                      */
    FA_B200_FLAG_NO_SPLIT = 16u        /* never divide the key axis of one (batch, head, query rows)
                                          problem among several CTAs.  By default the warp-specialised
                                          kernel may do so to keep every SM busy when the work items
                                          leave most SMs idle in the last round; the partial results
                                          are merged in fp32, in a fixed order, so a call repeats bit
                                          for bit, but where the cuts fall depends on how many
                                          (batch, head) pairs the call holds, and a divided problem
                                          differs from the undivided one by the kernel's ordinary
                                          rounding error.  With this flag the bits of one
                                          (batch, head) do not depend on what else is in the call (a
                                          shard reproduces the undivided job exactly)                */
};

/*
 * Launch the fused attention forward on `cuda_stream` (a cudaStream_t, NULL = default stream)
 * of CUDA device `device`.  Asynchronous unless FA_B200_FLAG_SYNC is given.
 *
 * Replaces the reference's launcher template
 *   launch_attention_kernel<head_dim, chunk_size>(B, L, F, q, k, v, mask, out, sync)
 * (include/fused_attn.cuh:860-894) together with the 12-way dispatch switch of
 * src/fused_attn_extention.cu:72-111.
 *
 * `chunk_hint` is validated with the reference's rules (power of two in [16,128], <= 2*head_dim,
 * not (16 with head_dim 128); src/fused_attn_extention.cu:45-47) so that existing callers see
 * the same rejections, but the tile sizes are internal and L need NOT be a multiple of it.
 * Pass 0 to skip the check.
 */
int fa_b200_attention_forward(const void* q, const void* k, const void* v,
                              const void* mask_or_null, void* y,
                              uint32_t B, uint32_t L, uint32_t F,
                              uint32_t head_dim, uint32_t chunk_hint,
                              int device, void* cuda_stream, uint32_t flags);

/*
 * Same operator with HOST buffers: copies q, k, v (and mask) to the device, runs the kernel and
 * copies y back, and returns when y is complete.  The work is cut into up to 8 chunks (batch
 * entries, or heads when B = 1) that flow through three internal streams, so the copy-in of one
 * chunk, the kernel of the previous and the copy-out of the one before overlap; pinned host
 * buffers are needed for that overlap.  Device staging buffers are cached per device and grow on
 * demand.  This is the call a torch-free
 * host program makes; it plays the role of the reference's standalone driver
 * (src/test.cu:43-62: cudaMalloc, fill, launch, synchronise).
 */
int fa_b200_attention_forward_host(const void* q, const void* k, const void* v,
                                   const void* mask_or_null, void* y,
                                   uint32_t B, uint32_t L, uint32_t F,
                                   uint32_t head_dim, uint32_t chunk_hint,
                                   int device, uint32_t flags);

/*
 * The same operator for callers that must not allocate.  It has no counterpart in the reference
 * (whose binding always allocates its output and whose launcher has no workspace at all).
 *
 * Who needs it: code that runs where cudaMalloc is off limits or unwanted: a process whose device
 * memory is entirely owned by another allocator or already handed out (an inference server that
 * reserves the whole GPU at start-up), a plugin that may not grow its host's footprint, a
 * latency-critical loop where an allocation would synchronise the device.
 * fa_b200_attention_forward allocates (once per device) a small status buffer for its kernels;
 * this entry point never calls cudaMalloc, cudaFree or any allocating library routine.
 *
 * How: it always runs the one-tile-per-CTA kernel, and that kernel's only scratch (a pair of
 * status words per CTA, written when a bounded device-side wait expires) lives in a fixed array
 * inside the library's device image: 16384 pairs = 128 KiB, held by every GPU that loads the
 * library until the process exits.  Consequences:
 *   - ceil(L/128) * (F/head_dim) * B must not exceed 16384 CTAs, otherwise the call is rejected
 *     with FA_B200_ERR_TOO_LARGE before anything is launched;
 *   - all calls on a device share that array.  Each call zeroes the pairs it is going to use (in
 *     stream order, ahead of its kernel) and the array otherwise keeps what the last call left;
 *     two calls whose kernels overlap on the GPU (different streams) race on it, so serialise them;
 *   - the first call on a device looks up the array's device address and sets the kernel's
 *     shared-memory attribute, two calls into the CUDA runtime that later calls do not make.
 *     Calls on different devices do not wait for one another.
 * flags: 0 or FA_B200_FLAG_SYNC (synchronise the stream and return FA_B200_ERR_DEVICE_TIMEOUT if
 * any CTA reported).  Inputs, outputs, head_dim, chunk_hint, mask: as fa_b200_attention_forward.
 */
int fa_b200_attention_forward_noalloc(const void* q, const void* k, const void* v,
                                      const void* mask_or_null, void* y,
                                      uint32_t B, uint32_t L, uint32_t F,
                                      uint32_t head_dim, uint32_t chunk_hint,
                                      int device, void* cuda_stream, uint32_t flags);

/*
 * Human-readable text for a status code returned by this library (negative codes) or by the
 * CUDA runtime (positive codes).  Replaces the stderr printing of the reference's
 * checkCudaError / checkLastCudaError (include/fused_attn.cuh:17-42).
 */
const char* fa_b200_strerror(int code);

/*
 * Device facts used by harnesses: out[0] = compute capability major, out[1] = minor,
 * out[2] = SM count, out[3] = max opt-in shared memory per block (bytes).
 * No counterpart in the reference (its CMake probes the device instead, CMakeLists.txt:12-39).
 */
int fa_b200_query(int device, int32_t out[4]);

/*
 * Read and clear the per-device status word written by kernels whose bounded waits expired:
 * out[0] = first failure code (0 = none; bits 8.. = role, bits 0..7 = barrier id),
 * out[1] = number of CTAs that reported.  Synchronises the device.
 * The word is shared by every launch on the device and stays set until it is read here, or
 * returned by a call with FA_B200_FLAG_SYNC or by fa_b200_attention_forward_host (both clear it
 * when they return FA_B200_ERR_DEVICE_TIMEOUT).  An asynchronous call never looks at it: after a
 * launch whose wait expired its output is garbage and only this word says so.  Once one CTA of a
 * launch has given up, the CTAs of that launch that start later leave at once.
 * No counterpart in the reference (it has no device-side error reporting).
 */
int fa_b200_read_status(int device, uint32_t out[2]);

/*
 * Exercise the bounded-wait path without touching the attention kernels: a one-warp kernel waits
 * (for about 10 ms) on a barrier that nothing completes, must give up, report and return.
 * out[0] = status code it recorded (expected 0x67F), out[1] = CTAs that reported (expected 1),
 * out[2] = 2 if the wait returned "gave up", 1 if it claimed success.  The GPU stays usable.
 * No counterpart in the reference (its kernels wait only on __syncthreads).
 */
int fa_b200_selftest_bounded_wait(int device, uint32_t out[3]);

/*
 * The checked build of the library (compiled with -DFA_DEBUG: every TMA copy and tensor-memory access
 * checks its shared-memory operand, its coordinates and its columns first, records a failed check in
 * the device status word and skips the access; tile buffers and Y are filled with NaN beforehand) can
 * test its own predicates: they are asked about operands that are in order and operands that are not,
 * with no copy made.  out[0] = status code recorded by the first refusal (expected 0x703: innermost
 * coordinate not a multiple of 8 elements), out[1] = 1, out[2] = 1 in a checked build and 0 in a normal
 * one (where nothing else is done), out[3] = one bit per predicate answered as it should be (expected
 * 0x7FF).  It plays the role of the reference's -g -G build of its smoke test (CMakeLists.txt:43) on
 * a pool where compute-sanitizer cannot be run.
 */
int fa_b200_selftest_debug_checks(int device, uint32_t out[4]);

#ifdef FA_CYCLES
/*
 * Only in the clock-counting build of the library (compiled with -DFA_CYCLES): from now on CTA 0 of the
 * warp-specialised kernels writes, per launch, four 64-bit words into record (launch id mod 64) of the
 * given device buffer of 256 words: the global timer (ns) at its entry, after its wait for the previous
 * kernel of the stream and at its end, and its SM clock count between the last two.  NULL stops the
 * recording.  The buffer must outlive the launches.  A build with -DFA_TIMELINE as well needs a buffer of
 * 9 * 1024 words: behind the 256, lane 0 of one warp per role of CTA 0 of the kernel on pairs of CTAs writes
 * its SM clock at up to eight events of each of the first 256 key steps (word 256 + (role * 256 + step) * 8 +
 * event; the roles and events are listed in csrc/fa_kernels.cuh and csrc/fa_pair.cuh).  No counterpart in the
 * reference.
 */
int fa_b200_debug_cycles(void* device_buffer_of_256_u64);
#endif

/*
 * Which kernel the default heuristics pick for a shape: returns 1 for the one-tile-per-CTA
 * kernel, 2 for the warp-specialised kernel, 3 for the warp-specialised kernel on pairs of CTAs
 * (head_dim 128, whole work items; a mask is taken to start on a 16-byte boundary, its rows then
 * do so whenever L is a multiple of 8), negative status on invalid arguments.
 * No counterpart in the reference.
 */
int fa_b200_select_kernel(uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                          int has_mask, uint32_t flags);

/*
 * How the warp-specialised kernel would spread a call's work over its CTAs on a device with
 * `sm_count` SMs: out[0] = kernel (1, 2 or 3, as fa_b200_select_kernel; for 3 a work item is 512 query
 * rows and out[1] CTAs form out[1]/2 pairs, nothing is divided), out[1] = CTAs launched,
 * out[2] = rounds of whole work items (a work item is 256 query rows of one (batch, head) against
 * all keys; CTA c takes items c, c + out[1], ...), out[3] = work items of the last, partial round
 * whose key steps are divided evenly among the first out[6] CTAs (0 = nothing is divided; a range
 * is at least half a work item, so a work item has at most three parts), out[4] = key steps of
 * those items in all, out[5] = key steps (tiles of 128 keys) per work item.  Pure arithmetic, no
 * CUDA call; it is what the launcher itself uses (FA_B200_FLAG_NO_SPLIT in `flags` is honoured).
 * No counterpart in the reference, whose grid is one CTA per (batch, query chunk, head)
 * (include/fused_attn.cuh:883).
 */
int fa_b200_describe_schedule(uint32_t B, uint32_t L, uint32_t F, uint32_t head_dim,
                              uint32_t flags, uint32_t sm_count, uint32_t out[7]);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
