/*
 * C ABI of the B200 (sm_100a) masked flash-attention forward.
 *
 * This is the boundary a host runtime binds: plain pointers and sizes, no C++
 * or torch types.  The reference has no C ABI for this path -- its launcher is a
 * header-only C++ template stack behind a torch operator -- so each entry point
 * below names the reference interface it stands in for.
 *
 * Conventions: every function returns FA_SM100_OK (0) or a negative
 * FA_SM100_ERR_* code, never throws, never synchronises the device (except
 * fa_mask_fwd_sm100_device_status, which says so) and never allocates device
 * memory: outputs and the workspace belong to the caller.  Work is enqueued on
 * the caller's stream.  (fa_mask_fwd_sm100 keeps two small blocks of pinned HOST memory,
 * allocated on first use: 64 bytes for the tile-skip heuristic described at
 * FaMaskFwdPlan.tile_skip and, per device, the word through which a kernel reports a wait
 * that gave up.  The first call on a device and for a kernel variant also sets function
 * attributes and looks up symbols: make it outside any stream capture.  While a stream is
 * being captured nothing is allocated; the heuristic and the report are then simply off.)
 *
 * Bounded waits: every wait inside the kernels has a limit (about a second).  A wait that
 * runs out makes its CTA drain and return, leaving `out` partly unwritten, and records a code
 * in a device status word and in the pinned host word.  Every later fa_mask_fwd_sm100 call on
 * that device then returns FA_SM100_ERR_DEVICE_WAIT without launching -- found by a plain host
 * load, no synchronisation -- until fa_mask_fwd_sm100_device_status(device, &st, 1) clears it.
 */
#ifndef FA_MASK_FWD_SM100_H_
#define FA_MASK_FWD_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_SM100_ABI_VERSION 2

enum {
    FA_SM100_OK = 0,
    FA_SM100_ERR_NULL = -1,        /* a required pointer is NULL */
    FA_SM100_ERR_DTYPE = -2,       /* dtype is neither FA_SM100_FP16 nor FA_SM100_BF16 */
    FA_SM100_ERR_SHAPE = -3,       /* negative size, Hk does not divide H, mask smaller than (Sq,Sk) */
    FA_SM100_ERR_HEAD_DIM = -4,    /* head_dim is neither 64 nor 128 */
    FA_SM100_ERR_ALIGN = -5,       /* q/k/v/out/workspace not 16-byte aligned */
    FA_SM100_ERR_WORKSPACE = -6,   /* workspace missing or smaller than workspace_bytes() says */
    FA_SM100_ERR_ARCH = -7,        /* the device is not compute capability 10.x */
    FA_SM100_ERR_CUDA = -8,        /* a CUDA runtime / driver call failed */
    FA_SM100_ERR_SPLITS = -9,      /* num_splits outside [0, FA_SM100_MAX_SPLITS] */
    FA_SM100_ERR_DEVICE_WAIT = -10,/* a kernel gave up on a bounded wait (see device_status) */
    FA_SM100_ERR_ABI = -11         /* struct_size does not match this library */
};

enum { FA_SM100_FP16 = 0, FA_SM100_BF16 = 1 };

/* Bits of FaMaskFwdArgs.disable.  Neither changes what is computed, only how. */
enum {
    FA_SM100_NO_TILE_SKIP = 1,  /* visit every key block even where the mask hides it entirely */
    FA_SM100_NO_UNIT_CUT = 2,   /* every (query pair, head, batch) unit is finished by one CTA, so the
                                 * result does not depend on the number of SMs */
    FA_SM100_NO_HEAD_PAIRS = 4, /* grouped-query heads are not paired: a unit is one head over a 256-row
                                 * query pair, as for ungrouped heads */
    FA_SM100_TEST_STALL_MASK = 0x100  /* tests only: the kernel's mask loads are withheld and its waits
                                 * get a short limit (FA_SM100_TEST_WAIT_KCYCLES in the environment,
                                 * units of 1024 SM cycles, default 2000), so that a wait runs out,
                                 * the kernel returns without writing `out` and the status paths can
                                 * be exercised without ever hanging a GPU */
};

#define FA_SM100_MAX_SPLITS 128

/*
 * Arguments of one forward call.  Field meanings follow the reference's
 * FA_mask_params (csrc/fa/common/fa_fwd_params.h:18-71) as filled by
 * mha_fwd_with_mask_cuda (csrc/fa/fa_fwd_op.cu:144-188): contiguous tensors
 *   q    (batch, heads,   seqlen_q, head_dim)
 *   k, v (batch, heads_k, seqlen_k, head_dim)
 *   mask (batch, 1, mask_seqlen_q >= seqlen_q, mask_seqlen_k >= seqlen_k)
 *   out  (batch, heads,   seqlen_q, head_dim)
 * all of the same 16-bit dtype.  The mask is additive (0 visible, -inf masked,
 * finite = bias), has no head dimension, and is addressed through its element
 * strides; columns >= seqlen_k are always masked whatever the mask holds there
 * and rows >= seqlen_q are never read.  The softmax scale is fixed at
 * 1/sqrt(head_dim).  Unlike the reference, seqlen_k and the mask pitch need no
 * multiple-of-8 padding by the caller (the reference pads K, V and the mask with
 * three copies, csrc/fa/fa_fwd_op.cu:117-138): K and V are read in place and only
 * a mask whose pitch or base breaks 16-byte row alignment is re-pitched into the
 * workspace.
 */
typedef struct FaMaskFwdArgs {
    uint32_t struct_size;       /* sizeof(FaMaskFwdArgs), checked */
    int32_t device;             /* CUDA device ordinal the pointers live on */
    const void* q;
    const void* k;
    const void* v;
    const void* mask;
    void* out;                  /* input dtype unless out_fp32 != 0 */
    float* lse;                 /* optional (batch, heads, seqlen_q) natural-log LSE, or NULL */
    int32_t batch;
    int32_t heads;
    int32_t heads_k;
    int32_t seqlen_q;
    int32_t seqlen_k;
    int32_t head_dim;
    int32_t mask_seqlen_q;
    int32_t mask_seqlen_k;
    int64_t mask_batch_stride;  /* elements */
    int64_t mask_row_stride;    /* elements */
    int32_t dtype;              /* FA_SM100_FP16 / FA_SM100_BF16 */
    int32_t num_splits;         /* 0 = choose, 1 = never split, n = force n KV splits */
    int32_t out_fp32;           /* 1: `out` is fp32 (normalised partial for a cross-GPU merge) */
    int32_t disable;            /* bit set of FA_SM100_NO_*: optimisations the caller switches off */
    uint64_t mask_version;      /* 0: nothing is remembered about the mask's content.  Otherwise a number
                                 * the caller changes whenever the content of this mask buffer changes:
                                 * the result of the tile-skip pre-pass is then kept inside the library,
                                 * per (mask pointer, strides, shape, dtype, device, version), and a
                                 * later call with the same key skips the pre-pass (and, where the mask
                                 * had nothing to skip, the skip list).  A caller that passes a stale
                                 * version gets results for the old content.  Ignored while the stream
                                 * is being captured, for a mask that has to be re-pitched (its copy
                                 * lives in the workspace) and by fa_mask_fwd_sm100_static_scratch. */
} FaMaskFwdArgs;

/* What the launcher decided for a set of arguments; for tests and tuning. */
typedef struct FaMaskFwdPlan {
    int32_t num_splits;         /* KV splits actually used (1 = single pass) */
    int32_t kv_blocks;          /* number of 128-key blocks */
    int32_t blocks_per_split;   /* largest split; split s owns blocks [s*nb/S, (s+1)*nb/S) */
    int32_t q_tiles_per_cta;    /* 128-row query tiles handled by one CTA */
    int32_t grid_x, grid_y, grid_z;   /* one-dimensional: grid_y = grid_z = 1 */
    int32_t threads;
    int32_t smem_bytes;
    int32_t mask_repitched;     /* 1 when the mask is first copied to an aligned pitch */
    int32_t sm_count;
    int32_t dual_split;         /* 1: one query tile per CTA, two KV splits side by side */
    int32_t tile_skip;          /* 1: eligible for tile skipping: a pre-pass kernel finds the key blocks
                                 * whose mask is -inf for a whole 256-row query pair (128-row tile with head_pairs) and the attention
                                 * kernel does not visit them (exact: their weights are 0).  The
                                 * launcher drops the pre-pass for a while after it found nothing to
                                 * skip twice in a row for the same mask buffer and shape. */
    int32_t unit_cut;           /* P >= 2: there are more single-pass units than CTAs and the R units
                                 * of the last, partial round are done by P <= SMs / R CTAs each (one
                                 * piece of the key blocks per CTA, merged through the workspace)
                                 * instead of leaving most SMs idle; 0: every unit is done by one CTA */
    int32_t head_pairs;         /* 1: grouped-query heads with an even group size: a unit is two heads of
                                 * one KV group over one 128-row query tile (they share every K/V tile
                                 * and every mask tile, and key blocks are skipped per 128 rows) */
    int32_t reserved0;
    uint64_t workspace_bytes;
} FaMaskFwdPlan;

/* Library / ABI version (FA_SM100_ABI_VERSION of the build). */
int fa_mask_fwd_sm100_abi_version(void);

/* Validates `args` and reports the launch plan without touching the device's
 * memory.  Replaces the policy half of fa_fwd_launch / fa_launch_sm8x
 * (csrc/fa/fa_fwd_launch.h:137-170, 262-309): split count, grid, workspace. */
int fa_mask_fwd_sm100_plan(const FaMaskFwdArgs* args, FaMaskFwdPlan* plan);

/* Bytes of scratch the call needs (0 is possible).  Replaces the per-call
 * torch::empty of the split-KV partial buffers (csrc/fa/fa_fwd_launch.h:289-297). */
int fa_mask_fwd_sm100_workspace_bytes(const FaMaskFwdArgs* args, size_t* bytes);

/* Enqueues the forward on `stream` (a cudaStream_t passed as void*).  Replaces
 * mha_fwd_with_mask_cuda's launch half and fa_fwd_launch
 * (csrc/fa/fa_fwd_op.cu:141-197, csrc/fa/fa_fwd_launch.h:573-603). */
int fa_mask_fwd_sm100(const FaMaskFwdArgs* args, void* workspace, size_t workspace_bytes,
                      void* stream);

/* Bytes of scratch built into the library for fa_mask_fwd_sm100_static_scratch. */
#define FA_SM100_STATIC_SCRATCH_BYTES (24u * 1024u * 1024u)

/* The same forward as fa_mask_fwd_sm100, for callers that have no way to hand over scratch
 * memory: code running where cudaMalloc is off limits (inside a region that is being captured
 * or replayed, in a latency-critical serving loop that forbids allocator calls, in a host
 * runtime whose memory pool is owned by someone else), or bindings that can only pass the
 * operator's own tensors.  It has no counterpart in the reference, whose launcher always
 * allocates its Split-KV buffers through torch (csrc/fa/fa_fwd_launch.h:289-297).
 *
 * Inputs and outputs are still the caller's.  The Split-KV partials, their LSE and a re-pitched
 * mask go into an array of FA_SM100_STATIC_SCRATCH_BYTES that is part of the library image, so
 * every GPU the library is loaded on holds that much until the process ends.  A call that
 * would need more returns FA_SM100_ERR_WORKSPACE and does nothing (a mask that must be
 * re-pitched counts in full: 4 x 1000 x 4104 elements, 32.8 MB, is already too much); nothing
 * is ever allocated or freed, by this function or by anything it calls.  Because the heuristic
 * that drops the tile-skip pre-pass keeps its state in pinned host memory, which this entry
 * point may not allocate, the pre-pass (a few microseconds) runs on every eligible call here,
 * also for masks that have nothing to skip; for the same reason a wait that gave up on the
 * device is reported to this entry point only once fa_mask_fwd_sm100 has set up the host word.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current) and keeps it; make that first call outside any stream capture.
 *
 * There is one array per device and every call uses it from its start: two calls whose GPU
 * work can overlap (different streams, no ordering between them) race on it and corrupt each
 * other's result; calls on one stream are safe.  The array keeps whatever the last call left
 * there, and nothing in it has to start at zero: partials, LSE values, the re-pitched mask, the
 * tile-skip flags and the unit counter are written by the call before it reads them, and the
 * hand-over slots of the unit cutting are guarded by tags that are compared with a value
 * unique to each launch (stale bytes never equal it) and taken back by their reader. */
int fa_mask_fwd_sm100_static_scratch(const FaMaskFwdArgs* args, void* stream);

/* The forward for a mask that is given by rules instead of a tensor - the recipes callers build
 * their additive masks from (examples/custom_mask_demo.py:33-65) - so that no (B, 1, Sq, Sk) mask
 * exists in memory at all:  key j is visible to query row i when  lo < j <= hi,
 *   hi = min(limit - 1, causal ? i + Sk - Sq : +inf),   lo = window > 0 ? i + Sk - Sq - window : -1,
 *   limit = min(Sk, valid_lens[batch])  (Sk when valid_lens is NULL; a device array of `batch` ints).
 * Bit-identical to fa_mask_fwd_sm100 on the mask that fa_mask_build_sm100 writes for the same rules.
 * The mask fields of `args` are ignored (mask may be NULL); `lse` is honoured; one pass over the
 * keys whatever num_splits says.  `workspace`: FA_SM100_RULE_WORKSPACE_BYTES of device memory, 16-byte
 * aligned, that no other call uses until this one has finished - the counter the CTAs take their
 * units from (units differ in length under a rule; the call zeroes it on the stream with a
 * cudaMemsetAsync ahead of the kernel); NULL: every CTA takes a fixed
 * share of the units instead (slower where the lengths differ much).  The reference has no such
 * operator. */
#define FA_SM100_RULE_WORKSPACE_BYTES 16
int fa_mask_fwd_sm100_rule(const FaMaskFwdArgs* args, int32_t causal, int32_t window, const int32_t* valid_lens,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Writes an additive mask (0 visible, -inf masked) of shape (batch, 1, seqlen_q, pitch) straight
 * into device memory from the rules callers of the operator otherwise spell out with a handful
 * of tensor operations (the reference's recipes, examples/custom_mask_demo.py:33-65; there is no
 * counterpart in the reference's operator interface).  Key j is visible to query i of batch b when
 *     j < seqlen_k
 *     and (valid_lens == NULL or j < valid_lens[b])                      padding
 *     and (causal == 0 or j <= i + seqlen_k - seqlen_q)                  causal, right-aligned
 *     and (window <= 0 or j > i + seqlen_k - seqlen_q - window)          sliding window
 * `pitch` >= seqlen_k is the row length in elements; a multiple of 8 keeps every row 16-byte
 * aligned, so the forward reads the mask in place however ragged seqlen_k is (pass it as
 * mask_seqlen_k = mask_row_stride = pitch).  Columns >= seqlen_k are written as -inf.
 * `valid_lens` is a device pointer to `batch` int32 values, or NULL. */
int fa_mask_build_sm100(void* mask, int32_t batch, int32_t seqlen_q, int32_t seqlen_k, int32_t pitch,
                        int32_t dtype, int32_t causal, int32_t window, const int32_t* valid_lens,
                        int32_t device, void* stream);

/* Merges `num_parts` normalised fp32 partial results that cover disjoint key
 * ranges: out = sum_s exp(lse_s - max) * o_s / sum_s exp(lse_s - max), rows whose
 * every lse is -inf give 0.  `o_parts` is (num_parts, rows, head_dim) fp32,
 * `lse_parts` (num_parts, rows) fp32, `out` (rows, head_dim) of `dtype`, or fp32
 * when out_fp32 != 0; `lse_out` (rows) is optional.  Same maths as the reference
 * combine kernel (csrc/fa/sm89/fa_fwd_kernel.h:1406-1545); exported so a
 * cross-GPU Split-KV can merge gathered partials. */
int fa_mask_fwd_sm100_combine(const float* o_parts, const float* lse_parts, void* out,
                              float* lse_out, int32_t num_parts, int64_t rows, int32_t head_dim,
                              int32_t dtype, int32_t out_fp32, int32_t device, void* stream);

/* The same merge for parts that arrive packed, as one all-gather over the ranks of a cross-GPU
 * Split-KV delivers them: part s occupies `part_stride` floats starting at packed + s *
 * part_stride, first its (rows, head_dim) fp32 output, directly behind it its (rows) LSE values
 * (so part_stride >= rows * (head_dim + 1); a multiple of 4 keeps every part 16-byte aligned).
 * A rank writes its own part with FaMaskFwdArgs.out = part, .lse = part + rows * head_dim,
 * .out_fp32 = 1, and nothing has to be copied or re-packed between the forward, the
 * collective and the merge.  No counterpart in the reference, which has no distributed code. */
int fa_mask_fwd_sm100_combine_packed(const float* packed, int64_t part_stride, void* out, float* lse_out,
                                     int32_t num_parts, int64_t rows, int32_t head_dim, int32_t dtype,
                                     int32_t out_fp32, int32_t device, void* stream);

/* The same merge with the exchange built in, for ranks (one process per GPU of one box) whose
 * parts live in peer-addressable ("symmetric") memory: every rank holds a buffer of the same
 * layout, `part_table` is a DEVICE array of `world` pointers, entry r = the base of rank r's
 * buffer as this GPU addresses it; a part (layout as for fa_mask_fwd_sm100_combine_packed)
 * starts `part_offset` floats into a buffer, and `flag_offset` floats into it lie `world` 32-bit
 * flag words that start at 0.  The kernel stores `seq` (the same on every rank for one call,
 * growing by one per call, never 0) into word `rank` of every rank's flags, waits until all of
 * its own words show at least `seq` -- bounded like every wait of this library: after about a
 * second it gives up, reports through the status word and writes nothing -- and then merges
 * the parts, reading the other GPUs' memory directly with plain loads (no multicast, no
 * collective library).  A caller alternates between two part slots from call to call, so that
 * a rank that is one call ahead never overwrites a part another rank is still reading.
 * No counterpart in the reference. */
int fa_mask_fwd_sm100_combine_peers(const void* part_table, int64_t part_offset, int64_t flag_offset,
                                    int32_t rank, int32_t world, uint32_t seq, void* out, float* lse_out,
                                    int64_t rows, int32_t head_dim, int32_t dtype, int32_t out_fp32,
                                    int32_t device, void* stream);

/* Synchronises `device` and returns in *status the sticky device-side status
 * word: 0, or the code of the first bounded wait that ran out.  Clears it when
 * `clear` != 0.  No counterpart in the reference, whose kernels wait unbounded. */
int fa_mask_fwd_sm100_device_status(int32_t device, uint32_t* status, int32_t clear);

/* Number of GPU kernels this library has launched in this process so far (attention, merge,
 * mask re-pitch and tile-skip pre-pass kernels).  For benchmarks that must report how many of
 * the library's kernels ran in a timed region.  No counterpart in the reference. */
int fa_mask_fwd_sm100_launch_count(uint64_t* launches);

/* Text for a return code.  Stands in for the TORCH_CHECK messages of
 * csrc/fa/fa_fwd_op.cu:53-108 and csrc/fa/fa_fwd_launch.h:596-602. */
const char* fa_mask_fwd_sm100_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* FA_MASK_FWD_SM100_H_ */
