// Masked flash-attention forward for B200 (sm_100a) behind a C ABI.
//
//   O = softmax(Q K^T / sqrt(d) + M) V        (M additive: 0, -inf or a finite bias)
//
// A unit of work is up to two 128-row query tiles of one (batch, head) and a range
// of 128-key blocks.  The kernel is persistent: one CTA per SM works through its
// units in turn, and the loads and the first MMA of the next unit run under the
// epilogue of the current one.  Roles inside the CTA (12 warps):
//
//   warps 0-3   softmax group of query tile 0   (thread <-> query row)
//   warps 4-7   softmax group of query tile 1
//   warp  8     MMA issuer: one thread issues tcgen05.mma; also owns tensor memory
//   warp  9     TMA producer for Q, K, V tiles
//   warp 10     TMA producer for the mask tiles
//   warp 11     unit scheduler: decodes the next unit (and, with tile skipping, its
//               list of key blocks to visit) one unit ahead and publishes it in
//               shared memory for the other roles
//
// Everything the tensor cores and the softmax threads touch arrives through TMA
// into 128-byte-swizzled shared memory behind mbarrier rings: Q (resident), a
// ring of K/V tiles, and per query tile two 128x64 mask panels.  The softmax
// threads read their own mask row from the swizzled panel with 16-byte loads,
// which the swizzle makes bank-conflict free.
//
// Tensor memory (512 columns x 128 lanes of 32 bit):
//   [  0,128) S of tile 0 (fp32), its first 64 columns are re-used for P (16 bit)
//   [128,256) S / P of tile 1
//   [256,256+d) O of tile 0 (fp32)      [384,384+d) O of tile 1
//
// Per key block j the MMA thread issues S_t = Q_t K_j^T (operands in shared
// memory), the softmax group of tile t reads S_t from tensor memory, adds the
// mask, keeps a running reference maximum and row sum, writes P_t back to tensor
// memory in the input dtype, and the MMA thread issues O_t += P_t V_j with P as
// the tensor-memory operand.  The two tiles alternate, so one tile's softmax runs
// under the other tile's MMAs.  O is rescaled in tensor memory only when a row's
// maximum grew by more than 2^8; the final 1/sum normalisation makes that exact.
//
// Semantics follow the reference operator (csrc/fa/fa_fwd_op.cu:46-197 and the
// kernel family it launches, csrc/fa/sm89/fa_fwd_kernel.h:73-480): fp32
// accumulation, score = s*scale + mask, -inf mask => weight 0, a fully masked row
// gives 0, columns >= seqlen_k are masked whatever the mask holds, P is rounded
// to the input dtype before P V, row sums stay fp32.  Split-KV writes normalised
// fp32 partials plus a natural-log LSE and a second kernel merges them
// (csrc/fa/sm89/fa_fwd_kernel.h:1406-1545).

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "../../include/fa_mask_fwd_sm100.h"
#include "arch_targets.h"
#include "sm100_ptx.cuh"

namespace fa_sm100 {

constexpr int kBlockM = 128;          // query rows per tile
constexpr int kBlockN = 128;          // keys per block
constexpr int kSoftmaxThreads = 128;  // one softmax group
constexpr int kMmaWarp = 8;
constexpr int kTmaWarp = 9;
constexpr int kMaskWarp = 10;
constexpr int kThreads = 384;
// Register re-balancing.  The kernel starts with kLaunchRegs per thread (what 384 threads
// leave of the 64K-register file: the allocation is per scheduler, three warps each).
// setmaxnreg.inc can only take what setmaxnreg.dec released inside the same CTA, and it
// blocks until that is there, so the books must balance or the softmax warps wait forever.
constexpr int kLaunchRegs = 168;
constexpr int kSoftmaxRegs = 216;
constexpr int kOtherRegs = 64;        // warps 8-11: one warpgroup, which must ask for one common count
static_assert(8 * (kSoftmaxRegs - kLaunchRegs) <= 4 * (kLaunchRegs - kOtherRegs),
              "setmaxnreg.inc would ask for more registers than setmaxnreg.dec releases");
static_assert(kThreads * kLaunchRegs <= 65536, "launch register budget");
// The register file is split between the four schedulers of an SM, and warp w lives on
// scheduler w % 4: each scheduler holds two softmax warps and one helper warp, and its
// quarter of the file (512 registers per lane) must hold all three after the re-balancing.
static_assert(2 * kSoftmaxRegs + kOtherRegs <= 512,
              "a scheduler's quarter of the register file cannot hold its three warps");
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxListBlocks = 384;    // key blocks a CTA can keep a skip list for (Sk <= 49152)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 5.545177444479562f;   // 8 * ln 2: rescale when max grew > 2^8
constexpr uint32_t kPanelBytes = 128 * 64 * 2;            // 128 rows x 64 columns, 16 bit

// Status codes written to the device status word when a bounded wait runs out.
enum : uint32_t {
    kStTmaEmpty = 1, kStMmaQ = 2, kStMmaKv = 3, kStMmaP = 4, kStSoftmaxS = 5, kStSoftmaxO = 6,
    kStDrain = 7, kStMaskEmpty = 8, kStSoftmaxMask = 9, kStList = 10, kStPartial = 11,
    kStPeer = 12     // the merge of a cross-GPU Split-KV waited in vain for another rank's part
};

__device__ unsigned int g_fa_status = 0;

template <int D>
struct Cfg {
    static constexpr int kStages = (D == 128) ? 3 : 6;            // K/V ring slots
    static constexpr uint32_t kTileBytes = kBlockM * D * 2;       // one Q, K or V tile
    static constexpr uint32_t kSubBytes = kPanelBytes;            // 64-column swizzle panel
    static constexpr int kSub = D / 64;
    static constexpr uint32_t kMaskBytes = 4 * kPanelBytes;       // 2 tiles x 2 panels
    static constexpr uint32_t kBarBytes = 512;            // mbarriers, small words, two unit boards
    static constexpr uint32_t kListBytes = 2 * kMaxListBlocks * 2;   // two compacted key-block lists (uint16)
    static constexpr uint32_t kSmemBytes =
        1024 + 2 * kTileBytes + kStages * kTileBytes + kMaskBytes + kBarBytes + kListBytes;
    static_assert(kSmemBytes <= 227 * 1024, "more shared memory than a CTA can have");
};

struct KParams {
    void* out;
    float* lse;
    float* o_part;            // (splits, B, H, Sq, D) fp32 when num_splits > 1
    float* lse_part;          // (splits, B, H, Sq)
    unsigned int* status;
    int B, H, Hk, Sq, Sk;
    int num_splits, kv_blocks;
    int m_pairs;              // row groups per (batch, head): 256-row query pairs, or 128-row tiles
                              // with head_pairs
    int head_pairs;           // 1: the two slots of a unit are two heads of one KV group over the
                              // SAME 128 query rows (they share every K/V tile and every mask tile)
    int total_units;          // B * (H or H/2) * m_pairs * split_groups; a CTA takes every gridDim.x-th one
    int split_groups;         // CTAs along the split axis: num_splits, or ceil(num_splits/2) in dual mode
    int dual;                 // 1: one query tile, two KV splits per CTA
    unsigned int* unit_counter;         // with block_flags: units taken beyond the first of each CTA
    const unsigned char* block_flags;   // (B, m_pairs, kv_blocks): 0 = every key of the block is masked
                                        // (-inf) for all rows of the group -> skipped; NULL = no skipping
    float* cut_part;          // per CTA: [256][D] fp32 O, then per CTA [256] LSE, then per CTA 8 tags
    unsigned long long cut_tag;   // value a softmax warp stores in its tag once its partial is written
    int cut_units;            // P >= 2: units of the last, partial round are done by P CTAs each; 0: whole
    int out_fp32;
    int wide_stores;          // 1: out and the partials are 32-byte aligned (256-bit stores)
    float scale;              // 1 / sqrt(d)
    unsigned int wait_kcycles;   // limit of every bounded wait, in units of 1024 SM cycles
    int mask_bcast;           // 1: one mask plane serves every batch element (batch stride 0)
    int test_stall_mask;      // test only: the mask producer loads nothing, so the waits for the
                              // mask run into their limit and the kernel reports it
    // RULE kernels: no mask tensor.  Key j is visible to query row i when
    //   lo < j <= hi,  hi = min(limit - 1, causal ? i + Sk - Sq : inf),  lo = window > 0 ? i + Sk - Sq - window : -1,
    //   limit = min(Sk, valid_lens[batch]) (Sk without valid_lens)
    // - the recipes of fa_mask_build_kernel, evaluated where they are used.
    // Units under a rule differ in length too: with `unit_counter` set the CTAs take them from it
    // (the launcher zeroes it on the stream before the kernel).
    int rule_causal, rule_window;
    const int* valid_lens;
};

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (BF16) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    } else {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (BF16) return pack_bf16x2(lo, hi);
    else return pack_f16x2(lo, hi);
}

// Unit cutting.  With G CTAs and units of equal length, whole rounds of G units go to the
// CTAs one unit each; the R < G units of a last, partial round would leave most SMs idle, so
// with P = G / R >= 2 each of them is done by P consecutive CTAs, one piece of its key blocks
// each.  Every piece but the last (kPartTail) ends in a normalised fp32 partial plus LSE in
// the CTA's slot of the workspace; the last piece (kPartHead), which the CTA with the highest
// index of the group holds, merges the partials of the other pieces into its own result.  The
// merging CTA is the one that is dispatched last: whatever it waits for was written by CTAs
// that are already resident or finished, also when another kernel holds part of the GPU.  (Equal shares of ALL steps, or of the last round's, were
// measured and lose: the partial traffic of 148 CTAs at once costs more than the idle SMs.)
enum : int { kPartWhole = 0, kPartTail = 1, kPartHead = 2 };

// Unit board: what the scheduler warp publishes about one unit of work, a (split group,
// 256-row query pair, head, batch) - or (split group, 128-row tile, pair of heads, batch) -
// combination, as ints in shared memory.  A CTA runs two
// softmax/MMA streams ("slots"); words kUiSlot + 4 * t + ... describe slot t.
enum : int {
    kUiB = 0, kUiH = 1, kUiSgroup = 2, kUiKvPlane = 3, kUiQPlane = 4,
    kUiUnit = 5,    // index of the unit; -1: no more work for this CTA
    kUiPart = 6,    // kPartWhole, kPartTail or kPartHead
    kUiPeerLast = 7,  // kPartHead: the first CTA that holds a piece of this unit (they end at this one)
    kUiSlot = 8,
    kUiSplit = 0,   // KV split the slot covers
    kUiBegin = 1,   // first key block
    kUiN = 2,       // key blocks to visit; 0: nothing visible; -1: the slot does not exist
    kUiRow0 = 3,    // first query row
    kUiInts = 16
};

// Epilogue helper.  Each softmax thread owns one output row, so a plain store instruction of
// a warp touches 32 different rows, 32 memory transactions of 16 or 32 bytes each, and the
// epilogue was bound by that.  Here the four lanes of a quad (four consecutive rows) first
// transpose 32-byte blocks among themselves: w[0..31] holds 128 contiguous bytes of the
// lane's own row on entry; on return w[8i..8i+7] holds block q = lane % 4 of the row of quad
// lane i.  Store i of the four lanes of a quad then writes one full 128-byte line of row i.
__device__ __forceinline__ void quad_transpose(uint32_t (&w)[32], int lane) {
    const bool odd1 = (lane & 1) != 0;
    const bool odd2 = (lane & 2) != 0;
    // step 1, partner lane ^ 1: of each pair of blocks (0,1) and (2,3) a lane keeps the one
    // with its own parity and swaps the other
#pragma unroll
    for (int b = 0; b < 4; b += 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t send = odd1 ? w[8 * b + i] : w[8 * (b + 1) + i];
            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
            if (odd1) w[8 * b + i] = recv;
            else w[8 * (b + 1) + i] = recv;
        }
    }
    // step 2, partner lane ^ 2: the same with the pairs of positions (0,1) and (2,3) as units
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t send = odd2 ? w[i] : w[16 + i];
        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 2);
        if (odd2) w[i] = recv;
        else w[16 + i] = recv;
    }
}

// Writes the transposed blocks: `row_ptr` = address of the 128-byte piece of the lane's OWN
// row, `row_bytes` = distance between consecutive rows, `rows_left` = valid rows counted from
// the lane's own row (<= 0: the lane's row is out of range).
__device__ __forceinline__ void quad_store(const uint32_t (&w)[32], int lane, char* row_ptr, long long row_bytes,
                                           int rows_left) {
    const int q = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i - q < rows_left) stg256(row_ptr + (i - q) * row_bytes + q * 32, &w[8 * i]);
}

// O *= alpha for the 32 rows of the calling warp (each thread its own row and factor).  Rare -
// a row's reference maximum moves a handful of times per unit - and therefore kept out of line,
// so that its few hundred instructions do not sit in the softmax loop's instruction stream.
template <int D>
__device__ __noinline__ void rescale_rows(uint32_t tO, float alpha) {
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(tO + c * 32, o);
    }
    tmem_wait_st();
}

// Cursor over a ring of mbarrier-guarded buffers: slot index and phase bit, advanced
// without any division.
struct Ring {
    int slot = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int slots) {
        if (++slot == slots) {
            slot = 0;
            phase ^= 1u;
        }
    }
};

template <int D, bool BF16, bool LIST, bool RULE = false>
__global__ void __launch_bounds__(kThreads, 1)
fa_mask_fwd_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_m,
                   const KParams p) {
    using C = Cfg<D>;
    constexpr int NS = C::kStages;
    constexpr uint32_t TILE = C::kTileBytes;
    constexpr uint32_t SUB = C::kSubBytes;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base = (raw_u32 + 1023u) & ~1023u;
    const uint32_t sQ = base;
    const uint32_t sKV = sQ + 2 * TILE;
    const uint32_t sM = sKV + NS * TILE;               // [slot][panel] of kPanelBytes
    const uint32_t sBar = sM + C::kMaskBytes;
    // mbarriers (8 bytes each)
    const uint32_t bar_q_full = sBar;                  // [2] Q tile landed
    const uint32_t bar_s_full = sBar + 16;             // [2] S of a slot computed
    const uint32_t bar_p_ready = sBar + 32;            // [2] first 64 keys of P written
    const uint32_t bar_o_full = sBar + 48;             // [2] last P.V of a unit done
    const uint32_t bar_m_full = sBar + 64;             // [4] mask panel landed
    const uint32_t bar_m_empty = sBar + 96;            // [4] mask panel consumed
    const uint32_t bar_kv_full = sBar + 128;           // [NS + 1] K/V ring (dual mode: one slot more)
    const uint32_t bar_kv_empty = sBar + 128 + 8 * (NS + 1);
    const uint32_t bar_p_ready2 = sBar + 240;          // [2] last 64 keys of P written
    const uint32_t bar_merge = sBar + 256;             // dual mode: both slots hold their final O
    const uint32_t bar_q_free = sBar + 264;            // [2] every S MMA that reads the Q tile is done
    const uint32_t bar_unit_full = sBar + 288;         // [2] unit board (and skip list) published
    const uint32_t bar_unit_empty = sBar + 304;        // [2] ... and no longer needed
    // small words, all addressed in the shared space (one register each, not two)
    const uint32_t tmem_slot_addr = sBar + 320;        // tensor-memory base written by tcgen05.alloc
    const uint32_t abort_flag = sBar + 324;            // set once a bounded wait of this CTA gave up
    const uint32_t bail_word = sBar + 328;
    const uint32_t wait_limit = sBar + 332;            // abort_flag + 8: limit of the bounded waits
    const uint32_t bar_scratch = sBar + 344;           // takes the arrivals of the softmax groups' first pass
    const uint32_t unit_board = sBar + 384;            // [2][kUiInts] ints
    const uint32_t blk_list = sBar + C::kBarBytes;     // [2][kMaxListBlocks] uint16

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Once any CTA of any launch gave up on a wait, the status word stays set until
    // the host clears it; later CTAs leave at once so a broken launch drains quickly.
    if (threadIdx.x == 0) {
        sts32(bail_word, *reinterpret_cast<volatile unsigned int*>(p.status));
        sts32(wait_limit, p.wait_kcycles);
    }
    __syncthreads();
    if (lds32(bail_word) != 0) return;

    // The CTA is persistent in pair mode: it takes units blockIdx.x, blockIdx.x + gridDim.x, ...
    // and every role keeps running counters for its barrier phases, so the producers and the
    // MMA thread run into the next unit (Q and K loads, first S = Q K^T) while the softmax
    // groups are still writing the previous unit's output.  Slots of a unit:
    //   pair mode  slot t = query tile t of the pair; both slots walk the same key blocks and
    //              share every K/V tile in shared memory;
    //   head pairs (pair mode with grouped-query heads, group size even) slot t = head 2u + t
    //              over the SAME 128 query rows: the slots share the K/V tiles and also the mask
    //              tile, which is loaded once for both, and key blocks are skipped per 128 rows;
    //   dual mode  (one query tile only, Split-KV; one unit per CTA) slot t = KV split
    //              2*group + t of the SAME query tile: two key ranges stream side by side.
    const bool dual = p.dual != 0;
    // dual mode needs one Q tile only: the second Q buffer becomes a fourth K/V ring slot
    const uint32_t ring_base = dual ? sKV - TILE : sKV;
    const int ring_slots = dual ? NS + 1 : NS;
    constexpr int kUnitConsumers = 3 + 8;   // two producers, MMA thread, lane 0 of each softmax warp

    // Decode of a unit and its publication on board k & 1 (scheduler warp, all lanes; see the
    // unit-scheduler role below).  The board is plain shared memory: the first unit of a CTA -
    // always unit blockIdx.x, whole - is decoded before the set-up barrier, under the tensor
    // memory allocation and the mbarrier initialisation of the other warps, and only its
    // arrival on the "full" mbarrier waits for that barrier.  (Not with a skip list: the block
    // flags are only valid once the pre-pass kernel has finished.)
    auto publish_unit = [&](int k, int unit, int part, int part_begin, int part_n, int peer_last) {
        int rest = unit;
        const int sgroup = rest % p.split_groups;
        rest /= p.split_groups;
        // later query rows first: under causal-like masks they carry the most key blocks
        const int mpair = p.m_pairs - 1 - (rest % p.m_pairs);
        rest /= p.m_pairs;
        const int heads_u = p.head_pairs ? (p.H >> 1) : p.H;
        const int h = p.head_pairs ? 2 * (rest % heads_u) : rest % heads_u;     // head of slot 0
        const int b = rest / heads_u;
        int count = 0;
        if constexpr (LIST) {
            const unsigned char* fl = p.block_flags +
                (static_cast<long long>(b) * p.m_pairs + mpair) * p.kv_blocks;
            const uint32_t lst = blk_list + (k & 1) * (kMaxListBlocks * 2);
            for (int base_j = 0; base_j < p.kv_blocks; base_j += 32) {
                const int jj = base_j + lane;
                const bool need = jj < p.kv_blocks && fl[jj] != 0;
                const unsigned ballot = __ballot_sync(0xffffffffu, need);
                if (need) sts16(lst + 2 * (count + __popc(ballot & ((1u << lane) - 1u))), static_cast<uint32_t>(jj));
                count += __popc(ballot);
            }
        }
        const uint32_t ui = unit_board + (k & 1) * (kUiInts * 4);
        if (lane < 2) {
            // lane t describes slot t
            const int t = lane;
            const int m0 = p.head_pairs ? mpair * kBlockM : mpair * (2 * kBlockM);
            const int split = dual ? 2 * sgroup + t : sgroup;
            // split s owns key blocks [s*nb/S, (s+1)*nb/S): sizes differ by at most one block
            const unsigned nb = static_cast<unsigned>(p.kv_blocks), ns = static_cast<unsigned>(p.num_splits);
            // (32 bits hold split * nb: at most 128 splits of at most 2^24 blocks)
            int begin = static_cast<int>(static_cast<unsigned>(split) * nb / ns);
            int end = static_cast<int>(static_cast<unsigned>(split + 1) * nb / ns);
            if (part != kPartWhole) {          // single pass, cut at a CTA boundary
                begin = part_begin;
                end = part_begin + part_n;
            }
            const int row0 = (dual || p.head_pairs) ? m0 : m0 + t * kBlockM;
            const bool on = dual ? (split < p.num_splits) : (row0 < p.Sq);
            if constexpr (RULE) {
                // the key blocks in which any row of the unit (both slots walk the same blocks)
                // sees a key: between the first row's lower limit and the last row's upper one
                const int rows = p.head_pairs ? kBlockM : 2 * kBlockM;
                const int r_last = min(m0 + rows, p.Sq) - 1;
                const int limit = p.valid_lens != nullptr ? min(p.Sk, p.valid_lens[b]) : p.Sk;
                const int hi = p.rule_causal ? min(limit - 1, r_last + p.Sk - p.Sq) : limit - 1;
                const int lo = p.rule_window > 0 ? m0 + p.Sk - p.Sq - p.rule_window : -1;
                begin = max(lo + 1, 0) / kBlockN;
                end = hi >= 0 ? hi / kBlockN + 1 : 0;
                if (end < begin) end = begin;
            }
            int n = on ? max(end - begin, 0) : -1;                 // -1: the slot does not exist
            if (LIST && on) n = count;                             // may be 0: nothing visible at all
            sts32(ui + 4 * (kUiSlot + 4 * t + kUiSplit), static_cast<uint32_t>(split));
            sts32(ui + 4 * (kUiSlot + 4 * t + kUiBegin), static_cast<uint32_t>(begin));
            sts32(ui + 4 * (kUiSlot + 4 * t + kUiN), static_cast<uint32_t>(n));
            sts32(ui + 4 * (kUiSlot + 4 * t + kUiRow0), static_cast<uint32_t>(row0));
            if (t == 0) {
                sts32(ui + 4 * (kUiUnit), static_cast<uint32_t>(unit));
                sts32(ui + 4 * (kUiPart), static_cast<uint32_t>(part));
                sts32(ui + 4 * (kUiPeerLast), static_cast<uint32_t>(peer_last));
                sts32(ui + 4 * (kUiB), static_cast<uint32_t>(b));
                sts32(ui + 4 * (kUiH), static_cast<uint32_t>(h));
                sts32(ui + 4 * (kUiSgroup), static_cast<uint32_t>(sgroup));
                sts32(ui + 4 * (kUiKvPlane), static_cast<uint32_t>(b * p.Hk + h / (p.H / p.Hk)));
                sts32(ui + 4 * (kUiQPlane), static_cast<uint32_t>(b * p.H + h));
            }
        }
    };
    // (The first unit of a CTA is unit blockIdx.x, whole, and can be decoded before the set-up
    // barrier - unless the launch has fewer units than CTAs, where every unit is cut in pieces.)
    const bool first_unit_whole = !(p.cut_units != 0 && p.total_units < static_cast<int>(gridDim.x));
    if (!LIST && first_unit_whole && warp == 11)
        publish_unit(0, static_cast<int>(blockIdx.x), kPartWhole, 0, p.kv_blocks, 0);

    if (warp == kTmaWarp && lane == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_q_full + 8 * t, 1);
            mbar_init(bar_s_full + 8 * t, 1);
            mbar_init(bar_p_ready + 8 * t, kSoftmaxThreads);
            mbar_init(bar_p_ready2 + 8 * t, kSoftmaxThreads);
            mbar_init(bar_o_full + 8 * t, 1);
            mbar_init(bar_q_free + 8 * t, 1);
            mbar_init(bar_unit_full + 8 * t, 1);
            mbar_init(bar_unit_empty + 8 * t, kUnitConsumers);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar_m_full + 8 * i, 1);
            // (with head pairs both softmax groups read panels 0 and 1)
            mbar_init(bar_m_empty + 8 * i, (p.head_pairs && i < 2) ? 2 * kSoftmaxThreads : kSoftmaxThreads);
        }
        for (int i = 0; i < NS + 1; ++i) {
            mbar_init(bar_kv_full + 8 * i, 1);
            mbar_init(bar_kv_empty + 8 * i, 1);
        }
        mbar_init(bar_merge, 2 * kSoftmaxThreads);
        mbar_init(bar_scratch, 0xfffffu);              // never completes a phase
        sts32(abort_flag, 0u);
        fence_barrier_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_m);
    }
    if (warp == kMmaWarp) {
        tmem_alloc(tmem_slot_addr, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = lds32(tmem_slot_addr);
    pdl_launch_dependents();      // a chained merge kernel may start its prologue now

    // Board of the k-th unit of this CTA (shared-space address); 0 when the wait gave up.
    auto unit_wait = [&](int k) -> uint32_t {
        if (!mbar_wait(bar_unit_full + 8 * (k & 1), (k >> 1) & 1, abort_flag, p.status, kStList)) return 0u;
        return unit_board + (k & 1) * (kUiInts * 4);
    };
    // word i of a board, as an int
    auto ui_get = [](uint32_t board, int i) -> int { return static_cast<int>(lds32(board + 4 * i)); };
    auto unit_done = [&](int k) { mbar_arrive(bar_unit_empty + 8 * (k & 1)); };

    if (warp >= 8) {
        // Data-movement and MMA-issue warps need few registers; hand the rest to softmax.
        // (setmaxnreg is a warpgroup-wide instruction: all four warps give the same count)
        reg_dealloc<kOtherRegs>();
        if (warp == kTmaWarp) {
            // -------------------------------------------------------------- Q/K/V producer
            if (lane == 0) {
                Ring ring;                      // next ring slot to fill, over all units
                int in_flight = 0;              // fills issued (capped), for the drain below
                uint32_t q_phase[2] = {1u, 1u}; // parity that says "Q tile t may be overwritten"
                bool ok = true;
                int kv_plane = 0;
                // One K or V tile into the next ring slot; false when a wait gave up.
                auto fill = [&](bool is_v, int block) -> bool {
                    // a fresh barrier passes the wait for the phase before its first one
                    if (!mbar_wait(bar_kv_empty + 8 * ring.slot, ring.phase ^ 1u, abort_flag, p.status,
                                   kStTmaEmpty))
                        return false;
                    const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
                    const uint32_t dst = ring_base + ring.slot * TILE;
                    const uint32_t bar = bar_kv_full + 8 * ring.slot;
                    mbar_arrive_expect_tx(bar, TILE);
#pragma unroll
                    for (int s = 0; s < C::kSub; ++s)
                        tma_load_3d(dst + s * SUB, tm, bar, s * 64, block * kBlockN, kv_plane);
                    ring.advance(ring_slots);
                    if (in_flight < ring_slots) ++in_flight;
                    return true;
                };
                int k = 0;
                for (; ok; ++k) {
                    const uint32_t ui = unit_wait(k);
                    if (!(ok = (ui != 0u)) || ui_get(ui, kUiUnit) < 0) break;
                    const uint32_t lst = blk_list + (k & 1) * (kMaxListBlocks * 2);
                    const int n0 = max(ui_get(ui, kUiSlot + kUiN), 0);
                    const int n1 = max(ui_get(ui, kUiSlot + 4 + kUiN), 0);
                    const int begin0 = ui_get(ui, kUiSlot + kUiBegin), begin1 = ui_get(ui, kUiSlot + 4 + kUiBegin);
                    const bool has_q1 = !dual && n1 > 0;
                    kv_plane = ui_get(ui, kUiKvPlane);
                    if (n0 > 0) {
                        const int q_plane = ui_get(ui, kUiQPlane);
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (!ok || (t == 1 && !has_q1)) continue;
                            // the tile may still be read by the previous unit's last S = Q K^T
                            if (!(ok = mbar_wait(bar_q_free + 8 * t, q_phase[t], abort_flag, p.status,
                                                 kStTmaEmpty)))
                                continue;
                            q_phase[t] ^= 1u;
                            mbar_arrive_expect_tx(bar_q_full + 8 * t, TILE);
#pragma unroll
                            for (int s = 0; s < C::kSub; ++s)
                                tma_load_3d(sQ + t * TILE + s * SUB, &tm_q, bar_q_full + 8 * t, s * 64,
                                            ui_get(ui, kUiSlot + 4 * t + kUiRow0),
                                            q_plane + (p.head_pairs ? t : 0));
                        }
                        if (!dual) {
                            // shared by both slots: K_0, V_0, K_1, V_1, ...
                            for (int j = 0; ok && j < n0; ++j) {
                                const int blk = LIST ? static_cast<int>(lds16(lst + 2 * j)) : begin0 + j;
                                ok = fill(false, blk) && fill(true, blk);
                            }
                        } else {
                            // the order the MMA thread consumes them: K_a0, K_b0, then per step
                            // V_a(j), K_a(j+1), V_b(j), K_b(j+1)
                            const int nmax = max(n0, n1);
                            ok = ok && fill(false, begin0);
                            if (ok && n1 > 0) ok = fill(false, begin1);
                            for (int j = 0; ok && j < nmax; ++j) {
                                if (ok && j < n0) ok = fill(true, begin0 + j);
                                if (ok && j + 1 < n0) ok = fill(false, begin0 + j + 1);
                                if (ok && j < n1) ok = fill(true, begin1 + j);
                                if (ok && j + 1 < n1) ok = fill(false, begin1 + j + 1);
                            }
                        }
                    }
                    unit_done(k);
                }
                if (lds32(abort_flag) != 0u) {
                    // Giving up: let the copies already in flight land before the CTA exits.
                    // Walk back over the last fills; the slot before `ring` was filled last.
                    Ring r = ring;
                    for (int i = 0; i < in_flight; ++i) {
                        if (r.slot == 0) {
                            r.slot = ring_slots;
                            r.phase ^= 1u;
                        }
                        --r.slot;
                        bool done = false;
                        for (uint32_t it = 0; it < kMaxPolls && !done; ++it)
                            done = mbar_try_wait(bar_kv_full + 8 * r.slot, r.phase);
                        if (!done) report_gave_up(p.status, kStDrain);
                    }
                }
            }
        } else if (warp == kMaskWarp) {
            // -------------------------------------------------------------- mask producer
            if (lane == 0) {
                // The mask may be a re-pitched copy written by the kernel launched just before
                // this one (chained with programmatic dependent launch): wait for it here, so
                // everything that does not need the mask has already started.
                pdl_wait_prior_grid();
                // Panel i = slot * 2 + half.  A slot's panels follow that slot's own key blocks.
                uint32_t ph[4] = {0u, 0u, 0u, 0u};      // phase of panel i's next load
                bool sent[4] = {false, false, false, false};
                bool ok = true;
                int k = 0;
                for (; ok; ++k) {
                    const uint32_t ui = unit_wait(k);
                    if (!(ok = (ui != 0u)) || ui_get(ui, kUiUnit) < 0) break;
                    const uint32_t lst = blk_list + (k & 1) * (kMaxListBlocks * 2);
                    const int n_of[2] = {max(ui_get(ui, kUiSlot + kUiN), 0), max(ui_get(ui, kUiSlot + 4 + kUiN), 0)};
                    const int begin_of[2] = {ui_get(ui, kUiSlot + kUiBegin), ui_get(ui, kUiSlot + 4 + kUiBegin)};
                    const int row0_of[2] = {ui_get(ui, kUiSlot + kUiRow0), ui_get(ui, kUiSlot + 4 + kUiRow0)};
                    const int b = p.mask_bcast ? 0 : ui_get(ui, kUiB);
                    const int nmax = (RULE || p.test_stall_mask) ? 0 : max(n_of[0], n_of[1]);
                    for (int j = 0; ok && j < nmax; ++j) {
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (!ok || j >= n_of[t]) continue;
                            if (t == 1 && p.head_pairs) continue;      // slot 1 reads slot 0's panels
                            const int blk = LIST ? static_cast<int>(lds16(lst + 2 * j)) : begin_of[t] + j;
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                const int i = 2 * t + hf;
                                if (!ok) continue;
                                if (!(ok = mbar_wait(bar_m_empty + 8 * i, ph[i] ^ 1u, abort_flag, p.status,
                                                     kStMaskEmpty)))
                                    continue;
                                mbar_arrive_expect_tx(bar_m_full + 8 * i, kPanelBytes);
                                tma_load_3d(sM + i * kPanelBytes, &tm_m, bar_m_full + 8 * i,
                                            blk * kBlockN + hf * 64, row0_of[t], b);
                                ph[i] ^= 1u;
                                sent[i] = true;
                            }
                        }
                    }
                    unit_done(k);
                }
                if (lds32(abort_flag) != 0u) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (!sent[i]) continue;
                        bool done = false;
                        for (uint32_t it = 0; it < kMaxPolls && !done; ++it)
                            done = mbar_try_wait(bar_m_full + 8 * i, ph[i] ^ 1u);
                        if (!done) report_gave_up(p.status, kStDrain);
                    }
                }
            }
        } else if (warp == 11) {
            // -------------------------------------------------------------- unit scheduler
            // Decodes the CTA's units one ahead of the roles that work on them and publishes
            // each on the unit board, so the integer divisions of the decode are paid once, off
            // every critical path.  With tile skipping (single-pass pair mode only) it also
            // compacts the unit's block flags - a pre-pass kernel marked the key blocks whose
            // mask is -inf for all 256 rows of a pair - into the list of blocks to visit.
            // Skipping such a block is exact: all of its weights are 0.
            if constexpr (LIST) pdl_wait_prior_grid();     // the flags come from the pre-pass kernel
            // Which unit comes next: a CTA starts with unit blockIdx.x; after that it takes every
            // gridDim.x-th one, or - with tile skipping, where units differ in length - the next
            // one nobody has taken yet, from a counter the pre-pass kernel reset.
            int unit = blockIdx.x;
            // unit cutting (see kPartWhole): whole rounds first, then one piece of a unit of the
            // last, partial round
            const int whole_rounds = p.total_units / static_cast<int>(gridDim.x);
            for (int k = 0;; ++k) {
                // board k&1 was last used by unit k-2: a fresh barrier passes at once
                const bool ok = mbar_wait(bar_unit_empty + 8 * (k & 1), ((k >> 1) & 1) ^ 1u, abort_flag,
                                          p.status, kStList);
                if (!__all_sync(0xffffffffu, ok)) break;
                int part = kPartWhole, part_begin = 0, part_n = p.kv_blocks, peer_last = 0;
                if (!LIST && p.cut_units) {
                    const int tail_unit = whole_rounds * static_cast<int>(gridDim.x) +
                                          static_cast<int>(blockIdx.x) / p.cut_units;
                    if (k < whole_rounds) {
                        unit = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
                    } else if (k > whole_rounds || tail_unit >= p.total_units) {
                        unit = p.total_units;
                    } else {
                        // CTAs c = u * P .. u * P + P - 1 share the u-th unit of the last round
                        const int piece = static_cast<int>(blockIdx.x) % p.cut_units;
                        unit = tail_unit;
                        // The last piece, the merging one, is one key block longer than its
                        // share: the other pieces' partials are then in memory by the time it
                        // wants them.
                        const int shift = p.kv_blocks >= 2 * p.cut_units ? 1 : 0;
                        part_begin = piece == 0 ? 0 : piece * p.kv_blocks / p.cut_units - shift;
                        part_n = (piece + 1 == p.cut_units ? p.kv_blocks
                                                           : (piece + 1) * p.kv_blocks / p.cut_units - shift) - part_begin;
                        part = piece + 1 == p.cut_units ? kPartHead : kPartTail;
                        peer_last = static_cast<int>(blockIdx.x) - (p.cut_units - 1);
                    }
                } else if (k > 0) {
                    if (LIST || (RULE && p.unit_counter != nullptr)) {
                        if (lane == 0) unit = static_cast<int>(gridDim.x + atomicAdd(p.unit_counter, 1u));
                        unit = __shfl_sync(0xffffffffu, unit, 0);
                    } else {
                        unit += gridDim.x;
                    }
                }
                if (unit >= p.total_units) {
                    if (lane == 0) {
                        sts32(unit_board + (k & 1) * (kUiInts * 4) + 4 * kUiUnit, 0xffffffffu);
                        mbar_arrive(bar_unit_full + 8 * (k & 1));
                    }
                    break;
                }
                if (LIST || k > 0 || !first_unit_whole) publish_unit(k, unit, part, part_begin, part_n, peer_last);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_unit_full + 8 * (k & 1));    // release: board and list visible
            }
        } else if (warp == kMmaWarp) {
            // -------------------------------------------------------------- MMA issuer
            if (lane == 0) {
                constexpr uint32_t idesc_s = make_idesc(BF16, false, kBlockM, kBlockN);
                constexpr uint32_t idesc_o = make_idesc(BF16, true, kBlockM, D);
                const uint32_t tS0 = tmem_base;
                const uint32_t tO0 = tmem_base + 256;
                Ring ring;                      // next K/V tile to take, in the producer's order
                uint32_t p_phase[2] = {0u, 0u}; // parity of slot t's next P hand-off
                uint32_t q_phase[2] = {0u, 0u}; // parity of Q tile t's next arrival
                bool ok = true;

                // S_t = Q_t K^T : A and B both K-major, 64-column 128B-swizzled panels.
                auto issue_s = [&](int t, uint32_t k_addr) {
                    uint32_t q_addr = dual ? sQ : sQ + t * TILE;   // dual: both slots share Q
                    // Built afresh at every call: left to itself the compiler keeps all of the
                    // loop-invariant Q descriptors in registers this warp does not have.
                    asm volatile("" : "+r"(q_addr));
                    const uint64_t da0 = smem_desc_sw128(q_addr, 16, 1024);
                    const uint64_t db0 = smem_desc_sw128(k_addr, 16, 1024);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        // the address field counts 16-byte units and cannot carry out of its bits
                        const uint32_t off16 = ((ks >> 2) * SUB + (ks & 3) * 32) >> 4;
                        mma_ss(tS0 + t * 128, da0 + off16, db0 + off16, idesc_s, ks > 0 ? 1u : 0u);
                    }
                };
                // O_t += P_t V : A = P in tensor memory (two 16-bit values per column),
                // B = V tile, d contiguous (MN-major), 16 keys per step.  P arrives in two
                // halves of 64 keys: the first half's MMAs run while the softmax threads are
                // still producing the second.
                auto issue_pv_half = [&](int t, uint32_t v_addr, bool acc, int half) {
                    const uint64_t dv0 = smem_desc_sw128(v_addr, SUB, 1024);
#pragma unroll
                    for (int kk = 0; kk < kBlockN / 32; ++kk) {
                        const int ks = half * (kBlockN / 32) + kk;
                        mma_ts(tO0 + t * 128, tS0 + t * 128 + ks * 8, dv0 + ((ks * 2048) >> 4), idesc_o,
                               (acc || ks > 0) ? 1u : 0u);
                    }
                };
                // waits for the two halves of P of the slot's next step and issues their MMAs;
                // `first` = first step of the unit (O is overwritten, not accumulated)
                auto issue_pv = [&](int t, uint32_t v_addr, bool first) -> bool {
                    if (!mbar_wait(bar_p_ready + 8 * t, p_phase[t], abort_flag, p.status, kStMmaP)) return false;
                    tc_fence_after();
                    issue_pv_half(t, v_addr, !first, 0);
                    if (!mbar_wait(bar_p_ready2 + 8 * t, p_phase[t], abort_flag, p.status, kStMmaP)) return false;
                    tc_fence_after();
                    issue_pv_half(t, v_addr, true, 1);
                    p_phase[t] ^= 1u;
                    return true;
                };
                auto wait_tile = [&](const Ring& r) -> bool {
                    return mbar_wait(bar_kv_full + 8 * r.slot, r.phase, abort_flag, p.status, kStMmaKv);
                };

                int k = 0;
                for (; ok; ++k) {
                    const uint32_t ui = unit_wait(k);
                    if (!(ok = (ui != 0u)) || ui_get(ui, kUiUnit) < 0) break;
                    const int n0 = max(ui_get(ui, kUiSlot + kUiN), 0);
                    const int n1 = max(ui_get(ui, kUiSlot + 4 + kUiN), 0);
                    unit_done(k);                // only the counts are needed here
                    if (n0 <= 0) continue;
                    if (!(ok = mbar_wait(bar_q_full, q_phase[0], abort_flag, p.status, kStMmaQ))) break;
                    q_phase[0] ^= 1u;
                    if (dual) {
                        // Two independent streams over a ring of NS + 1 slots; every K/V tile
                        // belongs to one slot and is released as soon as that slot's MMAs are
                        // issued.
                        const int n_of[2] = {n0, n1};
                        const int nmax = max(n0, n1);
                        auto release = [&]() {
                            mma_commit(bar_kv_empty + 8 * ring.slot);
                            ring.advance(NS + 1);
                        };
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (ok && n_of[t] > 0 && (ok = wait_tile(ring))) {
                                tc_fence_after();
                                issue_s(t, ring_base + ring.slot * TILE);
                                mma_commit(bar_s_full + 8 * t);
                                release();
                            }
                        }
                        for (int j = 0; ok && j < nmax; ++j) {
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                if (!ok || j >= n_of[t]) continue;
                                if (!(ok = wait_tile(ring))) continue;                    // V_t(j)
                                if (!(ok = issue_pv(t, ring_base + ring.slot * TILE, j == 0))) continue;
                                release();
                                if (j + 1 < n_of[t]) {
                                    if (!(ok = wait_tile(ring))) continue;                // K_t(j+1)
                                    tc_fence_after();
                                    issue_s(t, ring_base + ring.slot * TILE);
                                    mma_commit(bar_s_full + 8 * t);
                                    release();
                                } else {
                                    mma_commit(bar_o_full + 8 * t);
                                }
                            }
                        }
                        continue;
                    }
                    // ---- pair mode: K_j and V_j are shared by the two query tiles
                    const bool has_q1 = n1 > 0;
                    if (!(ok = wait_tile(ring))) break;                                   // K_0
                    tc_fence_after();
                    issue_s(0, sKV + ring.slot * TILE);
                    mma_commit(bar_s_full);
                    if (n0 == 1) mma_commit(bar_q_free);          // that was tile 0's last S
                    if (has_q1) {
                        if (!(ok = mbar_wait(bar_q_full + 8, q_phase[1], abort_flag, p.status, kStMmaQ))) break;
                        q_phase[1] ^= 1u;
                        tc_fence_after();
                        issue_s(1, sKV + ring.slot * TILE);
                        mma_commit(bar_s_full + 8);
                        if (n0 == 1) mma_commit(bar_q_free + 8);
                    }
                    mma_commit(bar_kv_empty + 8 * ring.slot);
                    ring.advance(NS);
                    for (int j = 0; ok && j < n0; ++j) {
                        const bool more = (j + 1) < n0;
                        const bool last_s = (j + 2) == n0;        // the S issued in this step is the unit's last
                        const Ring rv = ring;                     // V_j
                        Ring rk = ring;                           // K_{j+1}
                        rk.advance(NS);
                        const uint32_t v_addr = sKV + rv.slot * TILE;
                        const uint32_t k_addr = sKV + rk.slot * TILE;
                        if (!(ok = wait_tile(rv))) break;
                        // ---- tile 0
                        if (!(ok = issue_pv(0, v_addr, j == 0))) break;
                        if (more) {
                            if (!(ok = wait_tile(rk))) break;
                            tc_fence_after();
                            issue_s(0, k_addr);
                            mma_commit(bar_s_full);
                            if (last_s) mma_commit(bar_q_free);
                        } else {
                            mma_commit(bar_o_full);
                        }
                        // ---- tile 1
                        if (has_q1) {
                            if (!(ok = issue_pv(1, v_addr, j == 0))) break;
                            mma_commit(bar_kv_empty + 8 * rv.slot);
                            if (more) {
                                issue_s(1, k_addr);
                                mma_commit(bar_s_full + 8);
                                if (last_s) mma_commit(bar_q_free + 8);
                                mma_commit(bar_kv_empty + 8 * rk.slot);
                            } else {
                                mma_commit(bar_o_full + 8);
                            }
                        } else {
                            mma_commit(bar_kv_empty + 8 * rv.slot);
                            if (more) mma_commit(bar_kv_empty + 8 * rk.slot);
                        }
                        ring = rk;
                        if (more) ring.advance(NS);
                    }
                }
            }
        }
    } else {
        reg_alloc<kSoftmaxRegs>();
        // ------------------------------------------------------------------ softmax groups
        const int t = warp >> 2;
        const int wq = warp & 3;
        const int row_in_tile = wq * 32 + lane;
        const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + t * 128;
        const uint32_t tO = tmem_base + lane_sel + 256 + t * 128;
        const uint32_t bar_s = bar_s_full + 8 * t;
        const uint32_t bar_p = bar_p_ready + 8 * t;
        const uint32_t bar_p2 = bar_p_ready2 + 8 * t;
        // this thread's row inside a swizzled mask panel: 16-byte chunk c of row r
        // lives at r*128 + ((c ^ (r & 7)) << 4)
        const int mt = p.head_pairs ? 0 : t;             // whose mask panels this group reads
        const uint32_t m_row_addr = sM + (2 * mt) * kPanelBytes + row_in_tile * 128;
        const uint32_t m_xor = static_cast<uint32_t>(row_in_tile & 7) << 4;
        const float2 scale2 = make_float2(p.scale, p.scale);

        int gstep = 0;               // key-block steps of this slot so far, over all units
        int o_uses = 0;              // units of this slot that waited for their final O
        bool alive = true;
        // The body of a key-block step is some 15 KB of straight-line code, and a launch finds it
        // in no instruction cache: the first step of a CTA took about 12 000 cycles against 2300
        // for every later one (in-kernel cycle stamps), on the critical path of every CTA.  So the
        // loops below start with a pass "k = -1, j = -1" through that same code, without effect,
        // while the first loads are still on their way: its waits and arrivals go to a barrier
        // of their own that never completes a phase (a wait for the phase before a barrier's
        // first one passes at once), its stores to the O columns, which the unit's first P.V
        // overwrites, and its operands are whatever tensor and shared memory hold.  The pass is
        // told apart by address selects, not by branches around parts of the body: every form
        // with branches cost the steady-state loop more than the pass gains (measured).
        for (int k = -1; alive; ++k) {
            const bool warm = k < 0;
            const uint32_t ui = warm ? unit_board : unit_wait(k);
            if (!__all_sync(0xffffffffu, ui != 0u)) { alive = false; break; }
            if (!warm && ui_get(ui, kUiUnit) < 0) break;
            const uint32_t lst = blk_list + (k & 1) * (kMaxListBlocks * 2);
            const int n_t = warm ? 0 : ui_get(ui, kUiSlot + 4 * t + kUiN);
            if (n_t < 0) {                           // the slot does not exist in this unit
                __syncwarp();
                if (lane == 0) unit_done(k);
                continue;
            }
            const int begin_t = ui_get(ui, kUiSlot + 4 * t + kUiBegin);
            // RULE: the keys this thread's row sees, (rule_lo, rule_hi]
            int rule_lo = -1, rule_hi = 0x3fffffff;
            if constexpr (RULE) {
                if (!warm) {
                    const int bb = ui_get(ui, kUiB);
                    const int limit = p.valid_lens != nullptr ? min(p.Sk, p.valid_lens[bb]) : p.Sk;
                    const int diag = ui_get(ui, kUiSlot + 4 * t + kUiRow0) + row_in_tile + p.Sk - p.Sq;
                    rule_hi = p.rule_causal ? min(limit - 1, diag) : limit - 1;
                    rule_lo = p.rule_window > 0 ? diag - p.rule_window : -1;
                }
            }

            float m_ref = -INFINITY;     // reference maximum of the scaled, masked scores
            float l = 0.f;               // row sum relative to m_ref

            int j = warm ? -1 : 0;
            asm volatile("" : "+r"(j));  // (opaque: the first pass must stay inside the loop's code)
            for (; j < n_t; ++j) {
                const bool dummy = j < 0;
                const int col0 = (LIST ? static_cast<int>(lds16(lst + 2 * j)) : begin_t + j) * kBlockN;
                const bool tail = !dummy && (col0 + kBlockN) > p.Sk;
                const uint32_t par = (gstep & 1) ^ (dummy ? 1u : 0u);

                // The mask panels of this step were requested a whole step ago.  Their barriers
                // are tested first, while the scores are still being computed: a barrier test
                // costs about 150 cycles even when the barrier has long completed, and here that
                // latency falls into time the thread would spend waiting anyway, so that nothing
                // but the wake-up from the score barrier stands between S and the first load.
                bool ok = true;
                if constexpr (!RULE) {
                    ok = mbar_wait(dummy ? bar_scratch : bar_m_full + 8 * (2 * mt), par, abort_flag, p.status, kStSoftmaxMask);
                    ok = mbar_wait(dummy ? bar_scratch : bar_m_full + 8 * (2 * mt + 1), par, abort_flag, p.status, kStSoftmaxMask) && ok;
                }
                ok = mbar_wait(dummy ? bar_scratch : bar_s, par, abort_flag, p.status, kStSoftmaxS) && ok;
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                tc_fence_after();

                if (tail && !RULE) {
                    // Last key block of a ragged Sk: columns >= Sk are masked whatever the mask
                    // tile holds there.  Their scores are overwritten with -inf in tensor memory
                    // before the row is loaded (s * scale + mask is then -inf for any finite mask
                    // value), by a loop of single-column stores: a few instructions of code that
                    // run once per unit, where patching the values in registers took several
                    // hundred that sat in the middle of this loop's instruction stream.
#pragma unroll 1
                    for (int c = p.Sk - col0; c < kBlockN; ++c) tmem_st1(tS + c, 0xff800000u);
                    tmem_wait_st();
                }
                // pass 1: x = s*scale + mask for the whole 128-key block, block maximum
                uint32_t sreg[kBlockN];
                tmem_ld128(tS, sreg);
                float2 x[kBlockN / 2];
                float mt0 = -INFINITY, mt1 = -INFINITY;
                if constexpr (RULE) {
                    // No mask tile: the row sees the keys (rule_lo, rule_hi].  A block that every
                    // row of the warp sees entirely needs nothing but the scale; otherwise the
                    // row's 128 visibility bits are built from the two limits and each score gets
                    // 0 or -inf added (columns beyond Sk lie beyond rule_hi).
                    const int rel_lo = rule_lo - col0, rel_hi = rule_hi - col0;
                    const bool plain = __all_sync(0xffffffffu, rel_lo < 0 && rel_hi >= kBlockN - 1) && !dummy;
                    if (plain) {
                        const float2 zero2 = make_float2(0.f, 0.f);
#pragma unroll
                        for (int i = 0; i < kBlockN; i += 4) {
                            const float2 xa = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1])), scale2, zero2);
                            const float2 xb = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3])), scale2, zero2);
                            x[i / 2] = xa;
                            x[i / 2 + 1] = xb;
                            mt0 = max3(mt0, xa.x, xb.x);
                            mt1 = max3(mt1, xa.y, xb.y);
                        }
                    } else {
                        uint32_t vis[4];
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            // bits [a, b) of word w: keys col0 + 32 w + [a, b) are visible
                            const int a = min(max(rel_lo + 1 - 32 * w, 0), 32);
                            const int b = min(max(rel_hi + 1 - 32 * w, 0), 32);
                            const uint32_t below_b = b >= 32 ? 0xffffffffu : ((1u << b) - 1u);
                            const uint32_t below_a = a >= 32 ? 0xffffffffu : ((1u << a) - 1u);
                            vis[w] = b > a ? (below_b & ~below_a) : 0u;
                        }
#pragma unroll
                        for (int i = 0; i < kBlockN; i += 4) {
                            const uint32_t w = vis[i >> 5];
                            const int sh = i & 31;
                            const float2 a0 = make_float2(((w >> sh) & 1u) ? 0.f : -INFINITY,
                                                          ((w >> (sh + 1)) & 1u) ? 0.f : -INFINITY);
                            const float2 a1 = make_float2(((w >> (sh + 2)) & 1u) ? 0.f : -INFINITY,
                                                          ((w >> (sh + 3)) & 1u) ? 0.f : -INFINITY);
                            const float2 xa = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1])), scale2, a0);
                            const float2 xb = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3])), scale2, a1);
                            x[i / 2] = xa;
                            x[i / 2 + 1] = xb;
                            mt0 = max3(mt0, xa.x, xb.x);
                            mt1 = max3(mt1, xa.y, xb.y);
                        }
                    }
                } else {
#pragma unroll
                for (int pn = 0; pn < 2; ++pn) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 mv = lds128(m_row_addr + pn * kPanelBytes +
                                                ((static_cast<uint32_t>(c) << 4) ^ m_xor));
                        const uint32_t w[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                        for (int q = 0; q < 4; q += 2) {
                            const int i = pn * 64 + c * 8 + q * 2;        // column inside the block
                            const float2 xa = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1])),
                                scale2, unpack2<BF16>(w[q]));
                            const float2 xb = __ffma2_rn(
                                make_float2(__uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3])),
                                scale2, unpack2<BF16>(w[q + 1]));
                            x[i / 2] = xa;
                            x[i / 2 + 1] = xb;
                            mt0 = max3(mt0, xa.x, xb.x);
                            mt1 = max3(mt1, xa.y, xb.y);
                        }
                    }
                    mbar_arrive(dummy ? bar_scratch : bar_m_empty + 8 * (2 * mt + pn));      // panel may be refilled
                }
                }
                const float mt = fmaxf(mt0, mt1);

                // reference maximum moves only when the row maximum grew by more than 2^8
                const float m_new = fmaxf(m_ref, mt);
                const bool need = (m_new - m_ref) > kRescaleThreshold;  // NaN (-inf - -inf) -> false
                float alpha = 1.f;
                // A row that sees its first visible key only now has nothing worth rescaling in O
                // (at most the 1e-38 dust of the polynomial exponential times V, which vanishes
                // against the first real term), so it does not ask for the pass over O below.
                const bool rescale_o = need && (m_ref != -INFINITY);
                if (need) {
                    alpha = ex2((m_ref - m_new) * kLog2e);                // m_ref = -inf -> 0
                    m_ref = m_new;
                }
                if (j > 0 && __any_sync(0xffffffffu, rescale_o)) {
                    // PV of the previous block finished before this block's S was committed.
                    rescale_rows<D>(tO, alpha);
                }

                // pass 2: p = 2^((x - m_ref) * log2 e), fp32 row sum, P rounded to the input dtype
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                const float2 l2e2 = make_float2(kLog2e, kLog2e);
                const float2 nm2 = make_float2(-m_use * kLog2e, -m_use * kLog2e);
                float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const float2 e0 = __ffma2_rn(x[c * 16 + i], l2e2, nm2);
                        const float2 e1 = __ffma2_rn(x[c * 16 + i + 1], l2e2, nm2);
                        // bf16: three quarters of the exponentials go to the special-function
                        // unit, one quarter is computed on the FMA pipes (measured: +1.7 %; a
                        // larger share, or any share in the fp16 build, loses)
                        const float2 p0 = make_float2(ex2(e0.x), ex2(e0.y));
                        const float2 p1 = (BF16 && (i & 2)) ? ex2_poly2(e1) : make_float2(ex2(e1.x), ex2(e1.y));
                        sum_a = __fadd2_rn(sum_a, p0);
                        sum_b = __fadd2_rn(sum_b, p1);
                        pk[i] = pack2<BF16>(p0.x, p0.y);
                        pk[i + 1] = pack2<BF16>(p1.x, p1.y);
                    }
                    tmem_st16((dummy ? tO : tS) + c * 16, pk);
                    if (c == 1) {
                        // first 64 keys of P are in tensor memory: their MMAs may start
                        tmem_wait_st();
                        tc_fence_before();
                        mbar_arrive(dummy ? bar_scratch : bar_p);
                    }
                }
                l = l * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(dummy ? bar_scratch : bar_p2);
                gstep += dummy ? 0 : 1;
            }
            if (!alive) break;
            if (warm) continue;
            // the rest of the unit's description is read from the board only now, so that it
            // holds no registers during the loop above
            const int row = ui_get(ui, kUiSlot + 4 * t + kUiRow0) + row_in_tile;
            const bool row_ok = row < p.Sq;
            const int u_b = ui_get(ui, kUiB), u_sgroup = ui_get(ui, kUiSgroup);
            const int u_h = ui_get(ui, kUiH) + (p.head_pairs ? t : 0);
            const int split_t = ui_get(ui, kUiSlot + 4 * t + kUiSplit);
            const int n_other = ui_get(ui, kUiSlot + 4 * (t ^ 1) + kUiN);
            const int part = ui_get(ui, kUiPart);
            const int peer_last = ui_get(ui, kUiPeerLast);
            __syncwarp();
            if (lane == 0) unit_done(k);          // this warp no longer reads the board or the list

            // ---- epilogue: O / l, to the output dtype (or fp32 partial + LSE when split)
            // (a slot whose every key block was skipped has nothing in tensor memory: its rows
            // are fully masked, the result is 0 and the LSE -inf)
            const bool empty = (n_t == 0);
            if (!empty) {
                bool ok = mbar_wait(bar_o_full + 8 * t, o_uses & 1, abort_flag, p.status, kStSoftmaxO);
                ++o_uses;
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            }
            const bool merge_slots = dual && n_t > 0 && n_other > 0;
            if (merge_slots) {
                // Dual mode: the two slots hold partial results of the SAME rows over two key
                // ranges.  They are merged here, in the CTA, so one partial goes to memory
                // instead of two: each group publishes (max, sum) of its rows in its own, now
                // idle, mask panel, reads the other group's, and normalises half of the
                // columns of  a0*O0 + a1*O1  straight out of tensor memory.  (Dual mode runs
                // one unit per CTA, so the panel and the barrier are used once.)
                const uint32_t own = sM + (2 * t) * kPanelBytes + row_in_tile * 8;
                const uint32_t other = sM + (2 * (t ^ 1)) * kPanelBytes + row_in_tile * 8;
                sts32(own, __float_as_uint(m_ref));
                sts32(own + 4, __float_as_uint(l));
                mbar_arrive(bar_merge);
                bool ok = mbar_wait(bar_merge, 0, abort_flag, p.status, kStSoftmaxO);
                if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                tc_fence_after();
                const float m_o = __uint_as_float(lds32(other));
                const float l_o = __uint_as_float(lds32(other + 4));
                const bool dead_s = (m_ref == -INFINITY) || !(l > 0.f);
                const bool dead_o = (m_o == -INFINITY) || !(l_o > 0.f);
                const float m_all = fmaxf(dead_s ? -INFINITY : m_ref, dead_o ? -INFINITY : m_o);
                const float a_s = dead_s ? 0.f : __expf(m_ref - m_all);
                const float a_o = dead_o ? 0.f : __expf(m_o - m_all);
                const float l_all = a_s * l + a_o * l_o;
                const bool dead = dead_s && dead_o;
                const float inv = dead ? 0.f : 1.f / l_all;
                const float w_s = a_s * inv, w_o = a_o * inv;
                const long long prow =
                    ((static_cast<long long>(u_sgroup) * p.B + u_b) * p.H + u_h) * p.Sq + row;
                if (row_ok && t == 0) p.lse_part[prow] = dead ? -INFINITY : m_all + __logf(l_all);
                float* dst = p.o_part + prow * D;
                const uint32_t tO_other = tmem_base + lane_sel + 256 + (t ^ 1) * 128;
                constexpr int kChunks = D / 32;
#pragma unroll
                for (int cc = 0; cc < kChunks / 2; ++cc) {
                    const int c = t * (kChunks / 2) + cc;          // this group's half of the columns
                    uint32_t os[32], oo[32];
                    tmem_ld32(tO + c * 32, os);
                    tmem_ld32(tO_other + c * 32, oo);
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        os[i] = __float_as_uint(__uint_as_float(os[i]) * w_s + __uint_as_float(oo[i]) * w_o);
                    if (p.wide_stores) {
                        // quad-transposed, line-sized stores (see quad_transpose)
                        quad_transpose(os, lane);
                        quad_store(os, lane, reinterpret_cast<char*>(dst + c * 32), static_cast<long long>(D) * 4,
                                   p.Sq - row);
                    } else if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + c * 32 + i) =
                                make_float4(__uint_as_float(os[i]), __uint_as_float(os[i + 1]),
                                            __uint_as_float(os[i + 2]), __uint_as_float(os[i + 3]));
                    }
                }
            } else {
                tc_fence_after();
                // A row that never saw a visible key still has the reference maximum -inf; its
                // sum and accumulator hold only rounding dust of the polynomial exponential.
                const bool dead = (m_ref == -INFINITY) || !(l > 0.f);
                float inv = dead ? 0.f : (1.f / l);
                float lse_val = dead ? -INFINITY : m_ref + __logf(l);
                const int tile_row = t * kBlockM + row_in_tile;        // row inside the 256-row pair
                if (part == kPartHead) {
                    // The other pieces of this unit were done by the CTAs before this one, from peer_last on:
                    // in each, the softmax warp with the same rows wrote a normalised partial
                    // and then its tag.
                    const long long lse_base = static_cast<long long>(gridDim.x) * (2 * kBlockM) * D;
                    const unsigned long long* tags = reinterpret_cast<const unsigned long long*>(
                        p.cut_part + static_cast<long long>(gridDim.x) * (2 * kBlockM) * (D + 1));
                    for (int slot = peer_last; slot < static_cast<int>(blockIdx.x); ++slot) {
                        bool ok = true;
                        if (lane == 0) {
                            const long long t0 = clock64();
                            while (ld_acquire_u64(tags + slot * 8 + warp) != p.cut_tag) {
                                if (lds32(abort_flag) != 0u ||
                                    ((clock64() - t0) >> 10) > static_cast<long long>(p.wait_kcycles)) {
                                    ok = false;
                                    sts32(abort_flag, 1u);
                                    report_gave_up(p.status, kStPartial);
                                    break;
                                }
                            }
                        }
                        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
                        const float* part_o = p.cut_part + (static_cast<long long>(slot) * (2 * kBlockM) + tile_row) * D;
                        const float lse_p = ld_cg_f32(p.cut_part + lse_base + static_cast<long long>(slot) * (2 * kBlockM) +
                                                      tile_row);
                        // All loads of the partial are issued before the first is used (one at
                        // a time they cost a trip to the L2 each).  The four lanes of a quad read
                        // line-sized pieces of their four rows: the inverse of the stores below,
                        // see quad_transpose.
                        uint32_t pr[D];
                        const int q4 = lane & 3;
#pragma unroll
                        for (int c = 0; c < D / 32; ++c) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float* src = part_o + (i - q4) * D + c * 32 + q4 * 8;
                                const uint4 lo = ld_cg_v4(src), hi = ld_cg_v4(src + 4);
                                pr[c * 32 + 8 * i] = lo.x; pr[c * 32 + 8 * i + 1] = lo.y;
                                pr[c * 32 + 8 * i + 2] = lo.z; pr[c * 32 + 8 * i + 3] = lo.w;
                                pr[c * 32 + 8 * i + 4] = hi.x; pr[c * 32 + 8 * i + 5] = hi.y;
                                pr[c * 32 + 8 * i + 6] = hi.z; pr[c * 32 + 8 * i + 7] = hi.w;
                            }
                        }
                        // out = (a_o * O/l + a_p * o_p) / (a_o + a_p),  a = exp(lse - max lse);
                        // the merged, normalised row goes back to tensor memory
                        const float mx = fmaxf(lse_val, lse_p);
                        float w_o = 0.f, w_p = 0.f;
                        if (mx != -INFINITY) {
                            const float a_o = __expf(lse_val - mx), a_p = __expf(lse_p - mx);
                            const float den = a_o + a_p;
                            w_o = a_o / den * inv;
                            w_p = a_p / den;
                            lse_val = mx + __logf(den);
                        }
#pragma unroll
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t w[32], oc[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) w[i] = pr[c * 32 + i];
                            quad_transpose(w, lane);
                            tmem_ld32(tO + c * 32, oc);
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                oc[i] = __float_as_uint(__uint_as_float(oc[i]) * w_o + __uint_as_float(w[i]) * w_p);
                            tmem_st32(tO + c * 32, oc);
                        }
                        tmem_wait_st();
                        // The tag is taken back once the partial has been read (every load above
                        // has delivered its data), so a launch that repeats this one's tag - a
                        // replayed CUDA graph - cannot mistake this partial for its own.
                        __syncwarp();
                        if (lane == 0) st_release_u64(const_cast<unsigned long long*>(tags) + slot * 8 + warp, 0ull);
                        inv = 1.f;
                    }
                    if (!alive) break;
                }
                // the whole row is read from tensor memory with one load and one wait
                uint32_t o[D];
                if (!empty) {
                    if constexpr (D == 128) tmem_ld128(tO, o);
                    else tmem_ld64(tO, o);
                } else {
#pragma unroll
                    for (int i = 0; i < D; ++i) o[i] = 0u;
                }
                // where the row goes: the output, a Split-KV partial, or this CTA's cut partial
                const long long grow = (static_cast<long long>(u_b) * p.H + u_h) * p.Sq + row;
                float* o32 = nullptr;
                int rows_left = p.Sq - row;
                bool wide = p.wide_stores != 0;
                if (part == kPartTail) {
                    const long long slot = blockIdx.x;
                    o32 = p.cut_part + (slot * (2 * kBlockM) + tile_row) * D;
                    p.cut_part[static_cast<long long>(gridDim.x) * (2 * kBlockM) * D + slot * (2 * kBlockM) + tile_row] = lse_val;
                    rows_left = kBlockM;                  // every row of the slot exists
                    wide = true;                          // the workspace is 256-byte aligned
                } else if (p.num_splits > 1) {
                    // dual mode stores one partial per CTA (split group), otherwise one per split
                    const long long prow =
                        ((static_cast<long long>(dual ? u_sgroup : split_t) * p.B + u_b) * p.H + u_h) *
                            p.Sq + row;
                    o32 = p.o_part + prow * D;
                    if (row_ok) p.lse_part[prow] = lse_val;
                } else {
                    if (p.out_fp32) o32 = static_cast<float*>(p.out) + grow * D;
                    if (row_ok && p.lse != nullptr) p.lse[grow] = lse_val;
                }
                uint16_t* o16 = static_cast<uint16_t*>(p.out) + grow * D;
                if (wide) {
                    // quad-transposed, line-sized stores (see quad_transpose)
                    if (o32 != nullptr) {
#pragma unroll
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t w[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(o[c * 32 + i]) * inv);
                            quad_transpose(w, lane);
                            quad_store(w, lane, reinterpret_cast<char*>(o32 + c * 32), static_cast<long long>(D) * 4,
                                       rows_left);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < D / 64; ++c) {
                            uint32_t w[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                w[i] = pack2<BF16>(__uint_as_float(o[c * 64 + 2 * i]) * inv,
                                                   __uint_as_float(o[c * 64 + 2 * i + 1]) * inv);
                            quad_transpose(w, lane);
                            quad_store(w, lane, reinterpret_cast<char*>(o16 + c * 64), static_cast<long long>(D) * 2,
                                       rows_left);
                        }
                    }
                } else if (row_ok) {
                    // an output that is only 16-byte aligned: each thread stores its own row
                    if (o32 != nullptr) {
#pragma unroll
                        for (int i = 0; i < D; i += 4) {
                            float4 f;
                            f.x = __uint_as_float(o[i]) * inv;
                            f.y = __uint_as_float(o[i + 1]) * inv;
                            f.z = __uint_as_float(o[i + 2]) * inv;
                            f.w = __uint_as_float(o[i + 3]) * inv;
                            *reinterpret_cast<float4*>(o32 + i) = f;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < D; i += 8) {
                            uint4 uu;
                            uu.x = pack2<BF16>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                            uu.y = pack2<BF16>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                            uu.z = pack2<BF16>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                            uu.w = pack2<BF16>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                            *reinterpret_cast<uint4*>(o16 + i) = uu;
                        }
                    }
                }
                if (part == kPartTail) {
                    // publish: the partial rows of this warp, then its tag
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        unsigned long long* tag = reinterpret_cast<unsigned long long*>(
                            p.cut_part + static_cast<long long>(gridDim.x) * (2 * kBlockM) * (D + 1)) +
                            static_cast<long long>(blockIdx.x) * 8 + warp;
                        st_release_u64(tag, p.cut_tag);
                    }
                }
                // the next unit's first P.V overwrites O: every read above has completed
                // (tcgen05.wait::ld inside the loads), order it before the next arrivals
                tc_fence_before();
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------
// Split-KV merge: one warp per output row.
//   out = sum_s w_s o_s / sum_s w_s,  w_s = exp(lse_s - max_s lse_s)
// ---------------------------------------------------------------------------------
// Exchange of the parts of a cross-GPU Split-KV through peer memory.  Every rank keeps its
// part in a buffer that all ranks of the box can address (symmetric memory: the same layout on
// every rank, `parts[r]` = base of rank r's buffer as seen from this GPU).  The merge kernel of
// rank r first tells every rank "my part of call `seq` is complete" with one store into that
// rank's flag words, then waits - bounded - until its own flag words show `seq` from every
// rank, and then reads the other ranks' parts straight over NVLink with plain loads: no
// collective library call, no copy into local memory first.
struct PeerExchange {
    const float* const* parts;   // device array [world]; NULL: the parts are local (no exchange)
    long long part_offset;       // floats from a buffer's base to the part of this call
    long long flag_offset;       // floats from a buffer's base to its `world` flag words
    int rank, world;
    unsigned int seq;            // sequence number of this call, the same on every rank, never 0
    unsigned int wait_kcycles;   // limit of the wait, in units of 1024 SM cycles
    unsigned int* status;
};

__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int D>
__global__ void __launch_bounds__(256)
fa_mask_combine_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                       void* __restrict__ out, float* __restrict__ lse_out, int num_parts,
                       long long rows, int is_bf16, int out_fp32, long long o_part_stride,
                       long long lse_part_stride, const PeerExchange px) {
    constexpr int VEC = D / 32;
    const int lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // When chained behind the attention kernel with programmatic dependent launch, the
    // partials are only valid after this returns; otherwise it returns at once.
    pdl_wait_prior_grid();
    const bool peers = px.parts != nullptr;
    if (peers) {
        __shared__ int s_ok;
        if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < px.world) {
            // this rank's part was written by the kernels before this one in the stream
            __threadfence_system();
            unsigned int* f = reinterpret_cast<unsigned int*>(
                                  const_cast<float*>(px.parts[threadIdx.x]) + px.flag_offset) + px.rank;
            st_release_sys_u32(f, px.seq);
        }
        if (threadIdx.x == 0) {
            const unsigned int* mine = reinterpret_cast<const unsigned int*>(px.parts[px.rank] + px.flag_offset);
            const long long t0 = clock64();
            int ok = 1;
            for (int r = 0; r < px.world && ok; ++r) {
                // (a rank that is already one call ahead shows a larger number: that is fine too)
                while (static_cast<int>(ld_acquire_sys_u32(mine + r) - px.seq) < 0) {
                    if (((clock64() - t0) >> 10) > static_cast<long long>(px.wait_kcycles)) {
                        ok = 0;
                        break;
                    }
                }
            }
            if (!ok) report_gave_up(px.status, kStPeer);
            s_ok = ok;
        }
        __syncthreads();
        if (!s_ok) return;
    }
    if (row >= rows) return;

    float lse_r[FA_SM100_MAX_SPLITS / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < FA_SM100_MAX_SPLITS / 32; ++c) {
        const int s = c * 32 + lane;
        lse_r[c] = -INFINITY;
        if (s < num_parts)
            lse_r[c] = peers ? ld_cg_f32(px.parts[s] + px.part_offset + rows * D + row)
                             : lse_parts[static_cast<long long>(s) * lse_part_stride + row];
        mx = fmaxf(mx, lse_r[c]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float mx_use = (mx == -INFINITY) ? 0.f : mx;
    float w_r[FA_SM100_MAX_SPLITS / 32];
    float wsum = 0.f;
#pragma unroll
    for (int c = 0; c < FA_SM100_MAX_SPLITS / 32; ++c) {
        w_r[c] = __expf(lse_r[c] - mx_use);            // exp(-inf) = 0 for empty parts
        wsum += w_r[c];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);

    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    // eight parts per round: the loads of a round are independent and all in flight together
#pragma unroll
    for (int c = 0; c < FA_SM100_MAX_SPLITS / 32; ++c) {
        if (c * 32 >= num_parts) break;
        for (int s2 = 0; s2 < 32; s2 += 8) {
            if (c * 32 + s2 >= num_parts) break;
            float w[8];
            float4 f[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int part = c * 32 + s2 + u;
                w[u] = __shfl_sync(0xffffffffu, w_r[c], s2 + u);       // same in every lane
                f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (part < num_parts && w[u] != 0.f) {
                    // (another GPU's memory is read past the L1: the same addresses carry new
                    // data every other call)
                    const float* src = (peers ? px.parts[part] + px.part_offset
                                              : o_parts + static_cast<long long>(part) * o_part_stride) +
                                       row * D + lane * VEC;
                    if constexpr (VEC == 4) {
                        if (peers) {
                            const uint4 g = ld_cg_v4(src);
                            f[u] = make_float4(__uint_as_float(g.x), __uint_as_float(g.y), __uint_as_float(g.z),
                                               __uint_as_float(g.w));
                        } else {
                            f[u] = __ldg(reinterpret_cast<const float4*>(src));
                        }
                    } else {
                        if (peers) {
                            f[u].x = ld_cg_f32(src);
                            f[u].y = ld_cg_f32(src + 1);
                        } else {
                            const float2 g = __ldg(reinterpret_cast<const float2*>(src));
                            f[u].x = g.x; f[u].y = g.y;
                        }
                    }
                } else {
                    w[u] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc[0] += w[u] * f[u].x;
                acc[1] += w[u] * f[u].y;
                if constexpr (VEC == 4) {
                    acc[2] += w[u] * f[u].z;
                    acc[3] += w[u] * f[u].w;
                }
            }
        }
    }
    const float inv = (wsum > 0.f) ? 1.f / wsum : 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] *= inv;

    if (out_fp32) {
        float* dst = static_cast<float*>(out) + row * D + lane * VEC;
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        else *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
    } else {
        uint16_t* dst = static_cast<uint16_t*>(out) + row * D + lane * VEC;
        if constexpr (VEC == 4) {
            uint2 u;
            u.x = is_bf16 ? pack_bf16x2(acc[0], acc[1]) : pack_f16x2(acc[0], acc[1]);
            u.y = is_bf16 ? pack_bf16x2(acc[2], acc[3]) : pack_f16x2(acc[2], acc[3]);
            *reinterpret_cast<uint2*>(dst) = u;
        } else {
            *reinterpret_cast<uint32_t*>(dst) =
                is_bf16 ? pack_bf16x2(acc[0], acc[1]) : pack_f16x2(acc[0], acc[1]);
        }
    }
    if (lse_out != nullptr && lane == 0)
        lse_out[row] = (wsum > 0.f) ? mx + __logf(wsum) : -INFINITY;
}

// ---------------------------------------------------------------------------------
// Tile-skip pre-pass: one CTA per (key block, region of 256 or 128 query rows, batch) decides whether the
// mask holds anything but -inf in that 256 x 128 region (only rows < Sq and columns < Sk
// count).  flag = 1: the block must be visited; 0: every weight in it would be 0.
// The mask rows are 16-byte aligned here (the launcher re-pitches otherwise).  A CTA stops
// reading at the first pass that saw a visible entry, so a mask without all-masked regions
// costs a few kilobytes per CTA.
// ---------------------------------------------------------------------------------
// per-launch tally of skippable regions and a ticket that finds the last CTA
__device__ unsigned int g_skip_count = 0;
__device__ unsigned int g_skip_ticket = 0;

__global__ void __launch_bounds__(256)
fa_mask_classify_kernel(const uint16_t* __restrict__ mask, long long bs, long long rs, int Sq, int Sk,
                        uint32_t neg_inf2, unsigned char* __restrict__ flags, int* hint,
                        unsigned int* unit_counter, int region_rows) {
    const int nt = blockIdx.x, mp = blockIdx.y, b = blockIdx.z;
    pdl_wait_prior_grid();                          // a re-pitch kernel may have written the mask
    pdl_launch_dependents();
    // the attention kernel behind this one hands out its units from this counter
    if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x) == 0) *unit_counter = 0u;
    const int vec = threadIdx.x & 15;               // 16 vectors of 8 keys per 128-key row piece
    const int rsub = threadIdx.x >> 4;              // 16 rows per pass
    const int col = nt * kBlockN + vec * 8;
    const uint16_t neg_inf = static_cast<uint16_t>(neg_inf2 & 0xffffu);
    int visible = 0;
    // A region is `region_rows` = 256 rows (a query pair) or 128 rows (a tile shared by a pair of
    // heads) of one key block.  Passes of 16 rows in two rounds: 4 passes, a block-wide vote (a
    // region with anything visible usually ends here), then the others with all their loads in
    // flight at once.  (One pass per vote made a fully masked region cost 16 round trips to memory.)
    auto scan = [&](auto passes_tag, int pass0) {
        constexpr int kPasses = decltype(passes_tag)::value;
        uint4 v[kPasses];
        bool in[kPasses];
#pragma unroll
        for (int u = 0; u < kPasses; ++u) {
            const int row = mp * region_rows + (pass0 + u) * 16 + rsub;
            in[u] = row < Sq && col < Sk;
            v[u] = make_uint4(neg_inf2, neg_inf2, neg_inf2, neg_inf2);
            if (in[u]) v[u] = __ldg(reinterpret_cast<const uint4*>(mask + b * bs + row * rs + col));
        }
#pragma unroll
        for (int u = 0; u < kPasses; ++u) {
            if (!in[u]) continue;
            if (col + 8 <= Sk) {
                visible |= (v[u].x != neg_inf2) | (v[u].y != neg_inf2) | (v[u].z != neg_inf2) | (v[u].w != neg_inf2);
            } else {
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint16_t x = static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
                    if (col + e < Sk && x != neg_inf) visible = 1;
                }
            }
        }
    };
    scan(std::integral_constant<int, 4>{}, 0);
    visible = __syncthreads_or(visible) ? 1 : 0;
    if (!visible) {
        if (region_rows > kBlockM) scan(std::integral_constant<int, 12>{}, 4);
        else scan(std::integral_constant<int, 4>{}, 4);
        visible = __syncthreads_or(visible) ? 1 : 0;
    }
    if (threadIdx.x == 0) {
        flags[(static_cast<long long>(b) * gridDim.y + mp) * gridDim.x + nt] = visible ? 1 : 0;
        // Tell the host whether this mask has regions worth skipping: the CTAs tally on the
        // device and the last one to finish writes the total, once, to a word of mapped
        // pinned host memory that the host reads on a later call without synchronising.
        // (Only a heuristic input: overlapping launches may blur the tally, never a result.)
        if (hint != nullptr) {
            if (!visible) atomicAdd(&g_skip_count, 1u);
            __threadfence();
            const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
            if (atomicAdd(&g_skip_ticket, 1u) == total - 1) {
                *reinterpret_cast<volatile int*>(hint) =
                    static_cast<int>(*reinterpret_cast<volatile unsigned int*>(&g_skip_count)) + 1;
                g_skip_count = 0;
                g_skip_ticket = 0;
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// Mask re-pitch: copies the (Sq, Sk) corner of each batch's mask to a pitch that is
// a multiple of 8 elements so every row starts on a 16-byte boundary.  Pad columns
// get 0; the attention kernel masks columns >= Sk itself.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
fa_mask_repitch_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int Sq, int Sk,
                       int pitch, long long src_bs, long long src_rs) {
    pdl_launch_dependents();
    const long long r = blockIdx.x;                  // b * Sq + row
    const int b = static_cast<int>(r / Sq);
    const int row = static_cast<int>(r % Sq);
    const uint16_t* s = src + b * src_bs + row * src_rs;
    uint16_t* d = dst + r * pitch;
    // One 16-byte vector of the destination per thread and step.  The source row starts on
    // any 2-byte boundary: its bytes are fetched as the two aligned 16-byte vectors around
    // them and shifted into place (the misalignment is the same for the whole row).
    const uintptr_t s_addr = reinterpret_cast<uintptr_t>(s);
    const unsigned mis = static_cast<unsigned>(s_addr & 15u);         // even, 0..14
    const uint4* s16 = reinterpret_cast<const uint4*>(s_addr - mis);
    const unsigned word_off = mis >> 2, bit_shift = (mis & 3u) * 8u;
    for (int c = threadIdx.x * 8; c < pitch; c += blockDim.x * 8) {
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (c < Sk) {
            const int valid = min(8, Sk - c);                         // elements wanted from the source
            const uint4 lo = __ldg(s16 + (c >> 3));
            // the second vector only when a wanted byte lies in it (never reads past the vector
            // that holds the row's last element)
            uint4 hi = make_uint4(0u, 0u, 0u, 0u);
            if (mis + 2u * valid > 16u) hi = __ldg(s16 + (c >> 3) + 1);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint32_t o[4];
            switch (word_off) {                                       // uniform over the CTA
                case 0:
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = __funnelshift_r(w[k], w[k + 1], bit_shift);
                    break;
                case 1:
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = __funnelshift_r(w[k + 1], w[k + 2], bit_shift);
                    break;
                case 2:
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = __funnelshift_r(w[k + 2], w[k + 3], bit_shift);
                    break;
                default:
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = __funnelshift_r(w[k + 3], k + 4 < 8 ? w[k + 4] : 0u, bit_shift);
                    break;
            }
            if (valid < 8) {                                          // pad columns are 0
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (2 * k >= valid) o[k] = 0u;
                    else if (2 * k + 1 >= valid) o[k] &= 0xffffu;
                }
            }
            out = make_uint4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<uint4*>(d + c) = out;
    }
}

// ---------------------------------------------------------------------------------
// Mask from rules (padding / causal / sliding window): one 16-byte vector per thread.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
fa_mask_build_kernel(uint16_t* __restrict__ mask, int Sq, int Sk, int pitch, uint32_t neg_inf16, int causal,
                     int window, const int* __restrict__ valid_lens) {
    const long long r = blockIdx.x;                   // b * Sq + i
    const int b = static_cast<int>(r / Sq);
    const int i = static_cast<int>(r % Sq);
    const int limit = valid_lens != nullptr ? min(Sk, valid_lens[b]) : Sk;
    const int diag = i + Sk - Sq;                     // last key a causal query sees
    const int hi = causal ? min(limit - 1, diag) : limit - 1;          // visible keys: (lo, hi]
    const int lo = window > 0 ? diag - window : -1;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= pitch) return;
    uint16_t* dst = mask + r * pitch + c;
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int j0 = c + 2 * k, j1 = j0 + 1;
        const uint32_t e0 = (j0 > lo && j0 <= hi) ? 0u : neg_inf16;
        const uint32_t e1 = (j1 > lo && j1 <= hi) ? 0u : neg_inf16;
        w[k] = e0 | (e1 << 16);
    }
    if (c + 8 <= pitch && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        for (int e = 0; e < 8 && c + e < pitch; ++e)
            dst[e] = static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
    }
}

// ---------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;

// Kernels launched by this library since it was loaded (for benchmarks that must count them).
static std::atomic<unsigned long long> g_launches{0};

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    unsigned int* status_ptr = nullptr;
    unsigned int* status_host = nullptr;     // pinned, mapped: the kernels' copy of a wait that gave up
    bool status_host_failed = false;
    bool attr_set[12] = {false, false, false, false, false, false, false, false, false, false, false, false};
    bool queried = false;
};
static DeviceInfo g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int dev) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != dev) {
            err = cudaSetDevice(dev);
            switched = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

static inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Every failed CUDA runtime call leaves through here: the error is cleared (a launch-time
// error must not poison the caller's next call) and, with FA_SM100_DEBUG set in the
// environment, named on stderr together with the source line that saw it.
static int cuda_failed(int line) {
    const cudaError_t err = cudaGetLastError();
    static const bool verbose = std::getenv("FA_SM100_DEBUG") != nullptr;
    if (verbose)
        std::fprintf(stderr, "fa_mask_fwd_sm100: CUDA error at line %d: %s\n", line, cudaGetErrorString(err));
    return FA_SM100_ERR_CUDA;
}

static int validate(const FaMaskFwdArgs* a) {
    if (a == nullptr) return FA_SM100_ERR_NULL;
    if (a->struct_size != sizeof(FaMaskFwdArgs)) return FA_SM100_ERR_ABI;
    if (a->dtype != FA_SM100_FP16 && a->dtype != FA_SM100_BF16) return FA_SM100_ERR_DTYPE;
    if (a->head_dim != 64 && a->head_dim != 128) return FA_SM100_ERR_HEAD_DIM;
    if (a->batch < 0 || a->heads <= 0 || a->heads_k <= 0 || a->seqlen_q < 0 || a->seqlen_k < 0)
        return FA_SM100_ERR_SHAPE;
    if (a->heads % a->heads_k != 0) return FA_SM100_ERR_SHAPE;
    if (a->heads > 65535 || a->batch > 65535) return FA_SM100_ERR_SHAPE;
    if (a->mask_seqlen_q < a->seqlen_q || a->mask_seqlen_k < a->seqlen_k) return FA_SM100_ERR_SHAPE;
    if (a->mask_row_stride < a->mask_seqlen_k || a->mask_batch_stride < 0) return FA_SM100_ERR_SHAPE;
    // one mask plane for every batch element (stride 0) or planes that do not overlap
    if (a->batch > 1 && a->mask_batch_stride != 0 &&
        a->mask_batch_stride < static_cast<int64_t>(a->seqlen_q) * a->mask_row_stride)
        return FA_SM100_ERR_SHAPE;
    if (a->num_splits < 0 || a->num_splits > FA_SM100_MAX_SPLITS) return FA_SM100_ERR_SPLITS;
    if (a->device < 0 || a->device >= kMaxDevices) return FA_SM100_ERR_SHAPE;
    return FA_SM100_OK;
}

// SM count of the device, or the B200 figure where no device can be queried (the
// planner is also exercised on machines without a GPU).
static int query_device(int dev, DeviceInfo** out) {
    DeviceInfo& d = g_dev[dev];
    if (!d.queried) {
        int sms = 0, major = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess) {
            d.sm_count = sms;
            d.cc_major = major;
            d.queried = true;
        } else {
            cudaGetLastError();
            d.sm_count = 148;
            d.cc_major = 0;
        }
    }
    *out = &d;
    return FA_SM100_OK;
}

static bool mask_in_place(const FaMaskFwdArgs* a) {
    const int sk8 = (a->seqlen_k + 7) & ~7;
    // A NULL mask (planning before the buffers exist) counts as aligned.
    return (reinterpret_cast<uintptr_t>(a->mask) % 16 == 0) && (a->mask_row_stride % 8 == 0) &&
           (a->mask_batch_stride % 8 == 0) && (sk8 <= a->mask_row_stride);
}

// Scratch of the unit cutting: per CTA 256 rows of fp32 O, 256 LSE values and 8 tags.
static size_t cut_bytes(int ctas, int d) {
    return align256(static_cast<size_t>(ctas) * (2 * kBlockM) * (d + 1) * sizeof(float) +
                    static_cast<size_t>(ctas) * 8 * sizeof(unsigned long long));
}

// Tags of the unit cutting are unique per launch: a random start, then a counter.
static std::atomic<unsigned long long> g_cut_tag{0};
static unsigned long long next_cut_tag() {
    unsigned long long cur = g_cut_tag.load();
    if (cur == 0) {
        unsigned long long seed = static_cast<unsigned long long>(
            std::chrono::high_resolution_clock::now().time_since_epoch().count());
        seed ^= reinterpret_cast<uintptr_t>(&g_cut_tag) * 0x9E3779B97F4A7C15ull;
        seed = (seed * 0xBF58476D1CE4E5B9ull) | (1ull << 32);       // never 0
        g_cut_tag.compare_exchange_strong(cur, seed);
    }
    return g_cut_tag.fetch_add(1) + 1;
}

static int make_plan(const FaMaskFwdArgs* a, FaMaskFwdPlan* plan) {
    int rc = validate(a);
    if (rc != FA_SM100_OK) return rc;
    DeviceInfo* dev = nullptr;
    query_device(a->device, &dev);
    std::memset(plan, 0, sizeof(*plan));
    const int d = a->head_dim;
    int m_pairs = ceil_div(a->seqlen_q, 2 * kBlockM);
    const int nb = ceil_div(a->seqlen_k, kBlockN);
    const long long base_ctas = static_cast<long long>(m_pairs) * a->heads * a->batch;
    int splits = 1;
    if (nb > 0 && base_ctas > 0) {
        if (a->num_splits > 0) {
            splits = a->num_splits;
        } else if (base_ctas * 5 < static_cast<long long>(dev->sm_count) * 4 &&
                   nb >= (a->seqlen_q <= kBlockM ? 8 : 24)) {
            // Too few CTAs to fill the GPU: cut the key range so that about one CTA
            // lands on every SM, keeping at least four key blocks per CTA.  (With more than
            // one query tile a split costs a partial of 256 rows per CTA and a merge kernel
            // over all of them, about ten key blocks' time: measured, 64 units of 16 key
            // blocks take 52 us in two splits, 47 us whole and 45 us cut in two pieces that
            // the kernel merges itself - see unit_cut below - so short key ranges are not split.)
            const long long by_fill = dev->sm_count / base_ctas;
            const long long by_work = nb / 4;
            long long s = by_fill < by_work ? by_fill : by_work;
            if (s > FA_SM100_MAX_SPLITS) s = FA_SM100_MAX_SPLITS;
            if (s < 1) s = 1;
            splits = static_cast<int>(s);
        }
        if (splits > nb) splits = nb;
    }
    // One query tile and a split key range: a CTA takes two splits side by side (dual mode),
    // so aim for two splits per SM-filling CTA.
    const bool one_tile = a->seqlen_q <= kBlockM;
    if (one_tile && splits > 1 && a->num_splits == 0) {
        long long s2 = 2LL * splits;
        if (s2 > nb / 4) s2 = nb / 4;
        if (s2 > FA_SM100_MAX_SPLITS) s2 = FA_SM100_MAX_SPLITS;
        if (s2 > splits) splits = static_cast<int>(s2);
    }
    // split s owns blocks [s*nb/S, (s+1)*nb/S): never empty because S <= nb
    const int bps = nb > 0 ? ceil_div(nb, splits) : 0;
    const bool dual = one_tile && splits > 1;
    const int split_groups = dual ? ceil_div(splits, 2) : splits;
    // Grouped-query heads with an even group size: a unit is two heads of one group over one
    // 128-row tile instead of one head over two tiles.  K/V traffic is the same, every mask
    // tile is fetched once for two heads, and key blocks are skipped per 128 rows.
    const bool head_pairs = !dual && (a->heads / a->heads_k) % 2 == 0 &&
                            (a->disable & FA_SM100_NO_HEAD_PAIRS) == 0;
    if (head_pairs) m_pairs = ceil_div(a->seqlen_q, kBlockM);
    const int heads_u = head_pairs ? a->heads / 2 : a->heads;
    plan->num_splits = splits;
    plan->kv_blocks = nb;
    plan->blocks_per_split = bps;
    plan->q_tiles_per_cta = (a->seqlen_q > kBlockM || head_pairs) ? 2 : 1;
    plan->head_pairs = head_pairs ? 1 : 0;
    // Units of (split, 256-row query pair, head, batch), or (split, 128-row tile, pair of heads,
    // batch) with head_pairs.  Pair mode is persistent: one CTA per
    // SM takes every grid_x-th unit, so the loads and the first MMA of a unit run under the
    // previous unit's epilogue.  Dual mode runs one unit per CTA.  (Splitting the units of a
    // half-empty last round into single-tile CTAs was measured and gains nothing: a CTA's time
    // is set by the per-tile softmax -> MMA dependency chain, not by how many tiles it holds.)
    const long long units = static_cast<long long>(m_pairs) * split_groups * heads_u * a->batch;
    if (units > 0x3fffffffLL) return FA_SM100_ERR_SHAPE;
    plan->grid_x = static_cast<int32_t>((dual || units < dev->sm_count) ? units : dev->sm_count);
    plan->grid_y = 1;
    plan->grid_z = 1;
    plan->dual_split = dual ? 1 : 0;
    plan->threads = kThreads;
    plan->smem_bytes = static_cast<int32_t>(d == 128 ? Cfg<128>::kSmemBytes : Cfg<64>::kSmemBytes);
    plan->sm_count = dev->sm_count;
    plan->mask_repitched = (nb > 0 && a->seqlen_q > 0 && !mask_in_place(a)) ? 1 : 0;
    size_t ws = 0;
    const size_t rows = static_cast<size_t>(a->batch) * a->heads * a->seqlen_q;
    if (splits > 1) {
        // dual mode merges its two splits inside the CTA: one partial per split group
        ws += align256(static_cast<size_t>(split_groups) * rows * d * sizeof(float));
        ws += align256(static_cast<size_t>(split_groups) * rows * sizeof(float));
    }
    if (plan->mask_repitched) {
        const size_t pitch = (a->seqlen_k + 7) & ~7;
        ws += align256(static_cast<size_t>(a->batch) * a->seqlen_q * pitch * 2);
    }
    // Tile skipping: single pass over the keys, at least two key blocks, list fits the CTA.
    plan->tile_skip = (splits == 1 && nb >= 4 && nb <= kMaxListBlocks && a->seqlen_q > 0 &&
                       (a->disable & FA_SM100_NO_TILE_SKIP) == 0) ? 1 : 0;
    // (block flags, then the counter the attention kernel hands out its units from)
    if (plan->tile_skip) ws += align256(static_cast<size_t>(a->batch) * m_pairs * nb) + 256;
    // More single-pass units than CTAs and a last round that is at most half full: its units
    // are done in P pieces by P CTAs each.  A piece costs an epilogue of its own and the first
    // piece about 1.5 key blocks' time per partial it merges (measured), so the piece count
    // that pays is about sqrt(0.65 nb), and below six key blocks none does.
    // The same holds for a launch with fewer units than SMs, whose only round is a partial one
    // (a (batch, head) shard of a strong-scaled problem, a small batch): then every unit is cut
    // and the grid grows to units x pieces.
    // There a piece has to pay for itself against the whole unit, not against an idle SM: not
    // below twelve key blocks.
    plan->unit_cut = 0;
    if (!dual && splits == 1 && nb >= (units < dev->sm_count ? 12 : 6) && units > 0 &&
        units % dev->sm_count != 0 && (a->disable & FA_SM100_NO_UNIT_CUT) == 0) {
        long long pieces = dev->sm_count / (units % dev->sm_count);
        long long best = 2;
        while ((best + 1) * (best + 1) * 100 <= 65LL * nb) ++best;     // floor(sqrt(0.65 nb)), at least 2
        if (pieces > best) pieces = best;
        if (pieces >= 2) {
            plan->unit_cut = static_cast<int32_t>(pieces);
            if (units < dev->sm_count) plan->grid_x = static_cast<int32_t>(units * pieces);
        }
    }
    if (plan->unit_cut) ws += cut_bytes(plan->grid_x, d);
    plan->workspace_bytes = ws;
    return FA_SM100_OK;
}

static int get_encode() {
    if (g_encode != nullptr) return FA_SM100_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        return cuda_failed(__LINE__);
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return FA_SM100_OK;
}

// (planes, rows, cols) 16-bit tensor with element pitches `row_pitch` and `plane_pitch`,
// read in boxes of 128 rows x 64 columns with the 128-byte swizzle.
static int encode_map(CUtensorMap* tm, const void* ptr, int dtype, int planes, int rows, int cols,
                      long long row_pitch, long long plane_pitch) {
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                                static_cast<cuuint64_t>(planes)};
    // A single plane still needs a legal (multiple of 16 bytes, non-zero) outer stride.
    // (Callers pass planes = 1 for a mask whose one plane serves every batch element.)
    if (plane_pitch <= 0) plane_pitch = static_cast<long long>(rows) * row_pitch;
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_pitch) * 2,
                                   static_cast<cuuint64_t>(plane_pitch) * 2};
    const cuuint32_t box[3] = {64, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(
        tm, dtype == FA_SM100_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
        3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FA_SM100_OK : FA_SM100_ERR_CUDA;
}

// The four tensor maps depend only on pointers, shapes, pitches and dtype, not on data, and
// callers tend to come back with the same buffers (a layer called every step, a benchmark
// loop), so the last few sets are kept: encoding them costs several microseconds of host
// time per call, which is visible next to a 50 us kernel.
struct MapKey {
    const void* q; const void* k; const void* v; const void* mask;
    long long mask_rs, mask_bs;
    int dtype, B, H, Hk, Sq, Sk, d, device;
};
struct MapEntry {
    MapKey key;
    CUtensorMap tq, tk, tv, tm;
    bool valid = false;
};
constexpr int kMapCache = 8;
static MapEntry g_map_cache[kMapCache];
static int g_map_next = 0;
static std::mutex g_map_mutex;

static int get_maps(const MapKey& key, CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv,
                    CUtensorMap* tm) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    for (int i = 0; i < kMapCache; ++i) {
        const MapEntry& e = g_map_cache[i];
        if (e.valid && std::memcmp(&e.key, &key, sizeof(MapKey)) == 0) {
            *tq = e.tq; *tk = e.tk; *tv = e.tv; *tm = e.tm;
            return FA_SM100_OK;
        }
    }
    int rc;
    if ((rc = encode_map(tq, key.q, key.dtype, key.B * key.H, key.Sq, key.d, key.d,
                         static_cast<long long>(key.Sq) * key.d)) != FA_SM100_OK) return rc;
    if ((rc = encode_map(tk, key.k, key.dtype, key.B * key.Hk, key.Sk, key.d, key.d,
                         static_cast<long long>(key.Sk) * key.d)) != FA_SM100_OK) return rc;
    if ((rc = encode_map(tv, key.v, key.dtype, key.B * key.Hk, key.Sk, key.d, key.d,
                         static_cast<long long>(key.Sk) * key.d)) != FA_SM100_OK) return rc;
    // mask: (batch, Sq rows, Sk columns); reads beyond either extent return 0
    if ((rc = encode_map(tm, key.mask, key.dtype, key.mask_bs == 0 ? 1 : key.B, key.Sq, key.Sk, key.mask_rs,
                         key.mask_bs)) != FA_SM100_OK) return rc;
    MapEntry& e = g_map_cache[g_map_next];
    g_map_next = (g_map_next + 1) % kMapCache;
    e.key = key;
    e.tq = *tq; e.tk = *tk; e.tv = *tv; e.tm = *tm;
    e.valid = true;
    return FA_SM100_OK;
}

template <int D, bool BF16, bool LIST, bool RULE = false>
static int launch_fwd(DeviceInfo* dev, int slot, const CUtensorMap& tq, const CUtensorMap& tk,
                      const CUtensorMap& tv, const CUtensorMap& tm, const KParams& kp, dim3 grid,
                      cudaStream_t stream, bool chained) {
    auto kern = fa_mask_fwd_kernel<D, BF16, LIST, RULE>;
    if (!dev->attr_set[slot]) {
        // The in-kernel register re-balancing is only sound for the register count it was
        // written for; refuse to launch a build that came out different.
        cudaFuncAttributes fattr;
        if (cudaFuncGetAttributes(&fattr, kern) != cudaSuccess) return cuda_failed(__LINE__);
        if (fattr.numRegs != kLaunchRegs) {
            if (std::getenv("FA_SM100_DEBUG") != nullptr)
                std::fprintf(stderr, "fa_mask_fwd_sm100: kernel built with %d registers, expected %d\n",
                             fattr.numRegs, kLaunchRegs);
            return FA_SM100_ERR_CUDA;
        }
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(Cfg<D>::kSmemBytes)) != cudaSuccess) {
            return cuda_failed(__LINE__);
        }
        dev->attr_set[slot] = true;
    }
    if (chained) {
        // behind a pre-pass kernel: start this kernel's prologue under that kernel's tail
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = Cfg<D>::kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, tm, kp) != cudaSuccess) {
            return cuda_failed(__LINE__);
        }
        ++g_launches;
        return FA_SM100_OK;
    }
    kern<<<grid, kThreads, Cfg<D>::kSmemBytes, stream>>>(tq, tk, tv, tm, kp);
    if (cudaPeekAtLastError() != cudaSuccess) return cuda_failed(__LINE__);
    ++g_launches;
    return FA_SM100_OK;
}

static int launch_combine(const float* o_parts, const float* lse_parts, void* out, float* lse_out,
                          int parts, long long rows, int d, int dtype, int out_fp32,
                          cudaStream_t stream, bool chained = false, long long o_part_stride = 0,
                          long long lse_part_stride = 0, const PeerExchange* peer = nullptr) {
    if (rows <= 0) return FA_SM100_OK;
    PeerExchange px;
    std::memset(&px, 0, sizeof(px));
    if (peer != nullptr) px = *peer;
    // distance between consecutive parts, in floats; 0 = the parts follow one another
    if (o_part_stride == 0) o_part_stride = rows * d;
    if (lse_part_stride == 0) lse_part_stride = rows;
    const int warps = 8;
    const unsigned blocks = static_cast<unsigned>((rows + warps - 1) / warps);
    if (chained) {
        // Programmatic dependent launch behind the attention kernel: the launch latency
        // hides under that kernel's tail; the merge kernel waits on the grid dependency
        // before it reads a partial.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(warps * 32);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const int is_bf16 = dtype == FA_SM100_BF16;
        cudaError_t e = (d == 128)
            ? cudaLaunchKernelEx(&cfg, fa_mask_combine_kernel<128>, o_parts, lse_parts, out, lse_out,
                                 parts, rows, is_bf16, out_fp32, o_part_stride, lse_part_stride, px)
            : cudaLaunchKernelEx(&cfg, fa_mask_combine_kernel<64>, o_parts, lse_parts, out, lse_out,
                                 parts, rows, is_bf16, out_fp32, o_part_stride, lse_part_stride, px);
        if (e != cudaSuccess) {
            return cuda_failed(__LINE__);
        }
        ++g_launches;
        return FA_SM100_OK;
    }
    if (d == 128)
        fa_mask_combine_kernel<128><<<blocks, warps * 32, 0, stream>>>(
            o_parts, lse_parts, out, lse_out, parts, rows, dtype == FA_SM100_BF16, out_fp32,
            o_part_stride, lse_part_stride, px);
    else
        fa_mask_combine_kernel<64><<<blocks, warps * 32, 0, stream>>>(
            o_parts, lse_parts, out, lse_out, parts, rows, dtype == FA_SM100_BF16, out_fp32,
            o_part_stride, lse_part_stride, px);
    if (cudaPeekAtLastError() != cudaSuccess) return cuda_failed(__LINE__);
    ++g_launches;
    return FA_SM100_OK;
}

static int status_pointer(DeviceInfo* dev) {
    if (dev->status_ptr == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_fa_status) != cudaSuccess) {
            return cuda_failed(__LINE__);
        }
        dev->status_ptr = static_cast<unsigned int*>(ptr);
    }
    return FA_SM100_OK;
}

// A bounded wait that runs out leaves the output partly unwritten; the device status word
// records it, but reading that word means synchronising.  So the kernels also write the code
// to one word of pinned host memory mapped into the device's address space, and every forward
// looks at that word first - a plain host load, no synchronisation - and refuses to launch
// while it is set (fa_mask_fwd_sm100_device_status clears both).  The call that saw the
// timeout itself has already returned; it is the NEXT call that reports it.
// Allocating the word is skipped while `stream` is being captured (an allocation would break
// the capture) and where the caller must not allocate (`may_allocate` false).
static std::mutex g_status_host_mutex;
static void status_host_setup(DeviceInfo* dev, cudaStream_t stream, bool may_allocate) {
    if (dev->status_host != nullptr || dev->status_host_failed || !may_allocate) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    if (cap != cudaStreamCaptureStatusNone) return;
    std::lock_guard<std::mutex> lock(g_status_host_mutex);
    if (dev->status_host != nullptr || dev->status_host_failed) return;
    void* ptr = nullptr;
    if (cudaHostAlloc(&ptr, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        dev->status_host_failed = true;
        return;
    }
    *static_cast<volatile unsigned int*>(ptr) = 0u;
    void* dptr = nullptr;
    if (cudaHostGetDevicePointer(&dptr, ptr, 0) != cudaSuccess ||
        cudaMemcpyToSymbol(g_fa_status_host, &dptr, sizeof(dptr)) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeHost(ptr);
        dev->status_host_failed = true;
        return;
    }
    dev->status_host = static_cast<unsigned int*>(ptr);
}

// ---------------------------------------------------------------------------------
// Is the tile-skip pre-pass worth running for this mask?
// ---------------------------------------------------------------------------------
// The pre-pass costs a few microseconds and gates the attention kernel.  For a mask without
// any fully masked 256 x 128 region (an unstructured random mask) it buys nothing, so the
// launcher remembers, per mask buffer and shape, what the last pre-pass found: the pre-pass
// kernel counts the skippable regions into a word of mapped pinned host memory, which the
// host reads on a LATER call without synchronising anything.  Two pre-passes in a row that
// found nothing switch it off for the next kSkipHoldoff calls with that mask; then it is
// tried again, and every further miss doubles the pause up to kSkipHoldoffMax calls.  Only
// whether the optimisation runs depends on this; results never do.
constexpr int kHintSlots = 16;
constexpr int kSkipHoldoff = 30;
constexpr int kSkipHoldoffMax = 960;
struct SkipHint {
    const void* mask = nullptr;
    long long bs = 0, rs = 0;
    int B = 0, Sq = 0, Sk = 0, dtype = 0, device = 0;
    int zero_streak = 0;
    int holdoff = 0;
    int pause = kSkipHoldoff;     // length of the next pause
    bool ran_last = false;
    bool valid = false;
};
static SkipHint g_hints[kHintSlots];
static int g_hint_next = 0;
static int* g_hint_words = nullptr;          // kHintSlots ints, pinned + mapped
static bool g_hint_failed = false;
static std::mutex g_hint_mutex;

// Returns true when the pre-pass should run; *counter is where it should count (or NULL).
static bool want_classify(const FaMaskFwdArgs* a, const void* mask, long long bs, long long rs,
                          bool adaptive, cudaStream_t stream, int** counter) {
    *counter = nullptr;
    if (!adaptive) return true;
    std::lock_guard<std::mutex> lock(g_hint_mutex);
    if (g_hint_words == nullptr && !g_hint_failed) {
        // no allocation inside a stream capture: the pre-pass then simply runs
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
        if (cap != cudaStreamCaptureStatusNone) return true;
    }
    if (g_hint_words == nullptr && !g_hint_failed) {
        void* ptr = nullptr;
        if (cudaHostAlloc(&ptr, kHintSlots * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) !=
            cudaSuccess) {
            cudaGetLastError();
            g_hint_failed = true;
        } else {
            g_hint_words = static_cast<int*>(ptr);
            std::memset(g_hint_words, 0, kHintSlots * sizeof(int));
        }
    }
    if (g_hint_words == nullptr) return true;
    int slot = -1;
    for (int i = 0; i < kHintSlots; ++i) {
        const SkipHint& h = g_hints[i];
        if (h.valid && h.mask == mask && h.bs == bs && h.rs == rs && h.B == a->batch &&
            h.Sq == a->seqlen_q && h.Sk == a->seqlen_k && h.dtype == a->dtype && h.device == a->device) {
            slot = i;
            break;
        }
    }
    if (slot < 0) {
        slot = g_hint_next;
        g_hint_next = (g_hint_next + 1) % kHintSlots;
        SkipHint fresh;
        fresh.mask = mask; fresh.bs = bs; fresh.rs = rs; fresh.B = a->batch; fresh.Sq = a->seqlen_q;
        fresh.Sk = a->seqlen_k; fresh.dtype = a->dtype; fresh.device = a->device; fresh.valid = true;
        g_hints[slot] = fresh;
    }
    SkipHint& h = g_hints[slot];
    volatile int* word = g_hint_words + slot;
    if (h.holdoff > 0) {
        --h.holdoff;
        h.ran_last = false;
        return false;
    }
    if (h.ran_last) {
        // 0: the last pre-pass has not reported yet; 1: it found nothing to skip; > 1: it did
        if (*word == 1) {
            if (++h.zero_streak >= 2) {
                h.zero_streak = 0;
                h.holdoff = h.pause;
                h.pause = h.pause * 2 > kSkipHoldoffMax ? kSkipHoldoffMax : h.pause * 2;
                h.ran_last = false;
                return false;
            }
        } else if (*word > 1) {
            h.zero_streak = 0;
            h.pause = kSkipHoldoff;
        }
    }
    *word = 0;
    h.ran_last = true;
    *counter = g_hint_words + slot;            // unified addressing: same pointer on the device
    return true;
}

// ---------------------------------------------------------------------------------
// Block flags remembered across calls (FaMaskFwdArgs.mask_version != 0)
// ---------------------------------------------------------------------------------
// The pre-pass reads the whole mask again on every call although many callers present the same
// mask over and over (every layer of a model, every step of a benchmark).  The library cannot
// know that a buffer's content is unchanged, so it remembers flags only for callers that vouch
// for it with a version number they change when the content changes.  The flags live in a
// small static device array (no allocation), a handful of slots handed out round robin; each
// slot remembers its key, the stream and an event of the launch that filled it (a hit on
// another stream waits for that event), and an event of the last launch that read it (a slot
// is overwritten only behind that).  The pre-pass also tallies the regions it found skippable
// into a pinned host word: once that has arrived and says "none", hits run the plain kernel.
constexpr int kFlagSlots = 8;
constexpr size_t kFlagSlotBytes = 64 * 1024;
static __device__ __align__(256) unsigned char g_flag_cache[kFlagSlots][kFlagSlotBytes];
struct FlagEntry {
    const void* mask = nullptr;
    long long bs = 0, rs = 0;
    int B = 0, Sq = 0, Sk = 0, dtype = 0, device = 0, region_rows = 0;
    unsigned long long version = 0;
    bool valid = false;
    cudaStream_t fill_stream = nullptr;
    cudaEvent_t filled = nullptr, last_read = nullptr;
    bool read_recorded = false;
};
static FlagEntry g_flag_entries[kMaxDevices][kFlagSlots];      // per device: its own slots and events
static int g_flag_next[kMaxDevices] = {};
static int* g_flag_tally = nullptr;           // kMaxDevices * kFlagSlots ints, pinned + mapped
static void* g_flag_cache_addr[kMaxDevices] = {};
static std::mutex g_flag_mutex;

enum : int { kFlagsOff = 0, kFlagsFill = 1, kFlagsHit = 2, kFlagsHitNothing = 3 };
// Looks the key up.  kFlagsFill: *flags is a slot the caller must fill with the pre-pass on
// `stream` (tallying into *tally) and then seal with flag_cache_filled(); kFlagsHit: *flags holds
// valid flags (any cross-stream wait is already enqueued); kFlagsHitNothing: the mask is known
// to have nothing to skip; kFlagsOff: no caching for this call.
static int flag_cache_lookup(const FaMaskFwdArgs* a, const void* mask, long long bs, long long rs,
                             int region_rows, size_t flag_bytes, cudaStream_t stream, int* slot_out,
                             unsigned char** flags, int** tally) {
    *slot_out = -1;
    if (a->mask_version == 0 || flag_bytes > kFlagSlotBytes) return kFlagsOff;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
        cudaGetLastError();
        return kFlagsOff;
    }
    if (cap != cudaStreamCaptureStatusNone) return kFlagsOff;
    std::lock_guard<std::mutex> lock(g_flag_mutex);
    if (g_flag_tally == nullptr) {
        void* ptr = nullptr;
        if (cudaHostAlloc(&ptr, kMaxDevices * kFlagSlots * sizeof(int),
                          cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            return kFlagsOff;
        }
        g_flag_tally = static_cast<int*>(ptr);
        std::memset(g_flag_tally, 0, kMaxDevices * kFlagSlots * sizeof(int));
    }
    if (g_flag_cache_addr[a->device] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_flag_cache) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return kFlagsOff;
        }
        g_flag_cache_addr[a->device] = ptr;
    }
    unsigned char* base = static_cast<unsigned char*>(g_flag_cache_addr[a->device]);
    FlagEntry* entries = g_flag_entries[a->device];
    int* tallies = g_flag_tally + a->device * kFlagSlots;
    for (int i = 0; i < kFlagSlots; ++i) {
        FlagEntry& e = entries[i];
        if (e.valid && e.mask == mask && e.bs == bs && e.rs == rs && e.B == a->batch && e.Sq == a->seqlen_q &&
            e.Sk == a->seqlen_k && e.dtype == a->dtype && e.device == a->device &&
            e.region_rows == region_rows && e.version == a->mask_version) {
            // 0: the pre-pass has not reported yet; 1: nothing to skip; > 1: something
            if (*static_cast<volatile int*>(tallies + i) == 1) return kFlagsHitNothing;
            if (e.fill_stream != stream && cudaStreamWaitEvent(stream, e.filled, 0) != cudaSuccess) {
                cudaGetLastError();
                return kFlagsOff;
            }
            *slot_out = i;
            *flags = base + static_cast<size_t>(i) * kFlagSlotBytes;
            return kFlagsHit;
        }
    }
    const int i = g_flag_next[a->device];
    g_flag_next[a->device] = (i + 1) % kFlagSlots;
    FlagEntry& e = entries[i];
    if (e.filled == nullptr &&
        (cudaEventCreateWithFlags(&e.filled, cudaEventDisableTiming) != cudaSuccess ||
         cudaEventCreateWithFlags(&e.last_read, cudaEventDisableTiming) != cudaSuccess)) {
        cudaGetLastError();
        e.filled = nullptr;
        return kFlagsOff;
    }
    // whoever still reads the slot's old flags (possibly on another stream or device) goes first
    if (e.valid && e.read_recorded && cudaStreamWaitEvent(stream, e.last_read, 0) != cudaSuccess) {
        cudaGetLastError();
        return kFlagsOff;
    }
    e.valid = false;                      // sealed by flag_cache_filled()
    e.mask = mask; e.bs = bs; e.rs = rs; e.B = a->batch; e.Sq = a->seqlen_q; e.Sk = a->seqlen_k;
    e.dtype = a->dtype; e.device = a->device; e.region_rows = region_rows; e.version = a->mask_version;
    e.fill_stream = stream;
    e.read_recorded = false;
    tallies[i] = 0;
    *slot_out = i;
    *flags = base + static_cast<size_t>(i) * kFlagSlotBytes;
    *tally = tallies + i;
    return kFlagsFill;
}

static void flag_cache_filled(int device, int slot, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_flag_mutex);
    FlagEntry& e = g_flag_entries[device][slot];
    if (cudaEventRecord(e.filled, stream) == cudaSuccess) e.valid = true;
    else cudaGetLastError();
}

static void flag_cache_read(int device, int slot, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_flag_mutex);
    FlagEntry& e = g_flag_entries[device][slot];
    if (cudaEventRecord(e.last_read, stream) == cudaSuccess) e.read_recorded = true;
    else cudaGetLastError();
}

// A mask given by rules instead of a tensor (see KParams): what fa_mask_fwd_sm100_rule passes on.
struct RuleSpec {
    int causal, window;
    const int* valid_lens;
    unsigned int* counter;            // a word of device memory private to the launch, or NULL
};

static int forward(const FaMaskFwdArgs* a, void* workspace, size_t workspace_bytes,
                   cudaStream_t stream, bool adaptive_skip = true, const RuleSpec* rule = nullptr) {
    FaMaskFwdPlan plan;
    int rc = make_plan(a, &plan);
    if (rc != FA_SM100_OK) return rc;
    const long long rows = static_cast<long long>(a->batch) * a->heads * a->seqlen_q;
    if (rows == 0) return FA_SM100_OK;
    if (a->q == nullptr || a->out == nullptr) return FA_SM100_ERR_NULL;
    if (a->seqlen_k > 0 && (a->k == nullptr || a->v == nullptr || a->mask == nullptr))
        return FA_SM100_ERR_NULL;
    const uintptr_t align_or = reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) |
                               reinterpret_cast<uintptr_t>(a->v) | reinterpret_cast<uintptr_t>(a->out) |
                               reinterpret_cast<uintptr_t>(workspace);
    if (align_or % 16 != 0) return FA_SM100_ERR_ALIGN;
    if (plan.workspace_bytes > 0 && (workspace == nullptr || workspace_bytes < plan.workspace_bytes))
        return FA_SM100_ERR_WORKSPACE;

    DeviceGuard guard(a->device);
    if (guard.err != cudaSuccess) {
        return cuda_failed(__LINE__);
    }
    DeviceInfo* dev = nullptr;
    query_device(a->device, &dev);
    if (!dev->queried) return FA_SM100_ERR_CUDA;
    if (dev->cc_major != 10) return FA_SM100_ERR_ARCH;

    const int d = a->head_dim;
    if (a->seqlen_k == 0) {
        // No keys: every row is "fully masked" -> 0, LSE -inf.  A merge over zero parts
        // writes exactly that.
        return launch_combine(nullptr, nullptr, a->out, a->lse, 0, rows, d, a->dtype, a->out_fp32,
                              stream);
    }

    if ((rc = get_encode()) != FA_SM100_OK) return rc;
    if ((rc = status_pointer(dev)) != FA_SM100_OK) return rc;
    // (adaptive_skip is false exactly for the entry point that must not allocate)
    status_host_setup(dev, stream, /*may_allocate=*/adaptive_skip);
    if (dev->status_host != nullptr && *static_cast<volatile unsigned int*>(dev->status_host) != 0u)
        return FA_SM100_ERR_DEVICE_WAIT;

    // workspace carve-up: [o_part][lse_part][re-pitched mask]
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    float* o_part = nullptr;
    float* lse_part = nullptr;
    if (plan.num_splits > 1) {
        const int parts = plan.dual_split ? ceil_div(plan.num_splits, 2) : plan.num_splits;
        o_part = reinterpret_cast<float*>(ws);
        ws += align256(static_cast<size_t>(parts) * rows * d * sizeof(float));
        lse_part = reinterpret_cast<float*>(ws);
        ws += align256(static_cast<size_t>(parts) * rows * sizeof(float));
    }
    KParams kp;
    std::memset(&kp, 0, sizeof(kp));
    // The mask reaches the kernel through TMA, which wants a 16-byte aligned base and
    // pitches that are multiples of 16 bytes; anything else is re-pitched first.
    const uint16_t* mask_ptr = static_cast<const uint16_t*>(a->mask);
    long long mask_bs = a->mask_batch_stride;
    long long mask_rs = a->mask_row_stride;
    if (plan.mask_repitched) {
        const int pitch = (a->seqlen_k + 7) & ~7;
        uint16_t* dst = reinterpret_cast<uint16_t*>(ws);
        const unsigned blocks = static_cast<unsigned>(a->batch) * a->seqlen_q;
        fa_mask_repitch_kernel<<<blocks, 256, 0, stream>>>(
            mask_ptr, dst, a->seqlen_q, a->seqlen_k, pitch, mask_bs, mask_rs);
        if (cudaPeekAtLastError() != cudaSuccess) return cuda_failed(__LINE__);
        ++g_launches;
        mask_ptr = dst;
        mask_bs = static_cast<long long>(a->seqlen_q) * pitch;
        mask_rs = pitch;
    }
    int* hint_counter = nullptr;
    const int region_rows = plan.head_pairs ? kBlockM : 2 * kBlockM;
    const int regions = ceil_div(a->seqlen_q, region_rows);
    const size_t flag_bytes = static_cast<size_t>(a->batch) * regions * plan.kv_blocks;
    // (the remembered flags describe the caller's own buffer: not for a re-pitched copy, whose
    // address changes with the workspace, and not for the entry point that keeps no state)
    int flag_slot = -1;
    unsigned char* cached_flags = nullptr;
    const int cache = (plan.tile_skip && adaptive_skip && !plan.mask_repitched)
        ? flag_cache_lookup(a, mask_ptr, mask_bs, mask_rs, region_rows, flag_bytes, stream, &flag_slot,
                            &cached_flags, &hint_counter)
        : kFlagsOff;
    const bool run_classify = plan.tile_skip && cache != kFlagsHit && cache != kFlagsHitNothing &&
        (cache == kFlagsFill || want_classify(a, mask_ptr, mask_bs, mask_rs, adaptive_skip, stream, &hint_counter));
    unsigned char* ws_flags = ws + (plan.mask_repitched
        ? align256(static_cast<size_t>(a->batch) * a->seqlen_q * ((a->seqlen_k + 7) & ~7) * 2) : 0);
    unsigned int* ws_unit_counter = reinterpret_cast<unsigned int*>(ws_flags + align256(flag_bytes));
    if (cache == kFlagsHit) {
        // no pre-pass: its other job, resetting the counter the units are handed out from, is done here
        if (cudaMemsetAsync(ws_unit_counter, 0, sizeof(unsigned int), stream) != cudaSuccess) return cuda_failed(__LINE__);
        kp.block_flags = cached_flags;
        kp.unit_counter = ws_unit_counter;
    }
    if (run_classify) {
        unsigned char* flags = cache == kFlagsFill ? cached_flags : ws_flags;
        unsigned int* unit_counter = ws_unit_counter;
        const dim3 cgrid(plan.kv_blocks, regions, a->batch);
        const uint32_t ninf = a->dtype == FA_SM100_BF16 ? 0xFF80FF80u : 0xFC00FC00u;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = cgrid;
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = plan.mask_repitched ? 1 : 0;      // chained behind the re-pitch kernel
        if (cudaLaunchKernelEx(&cfg, fa_mask_classify_kernel, mask_ptr, mask_bs, mask_rs, a->seqlen_q,
                               a->seqlen_k, ninf, flags, hint_counter, unit_counter, region_rows) != cudaSuccess) {
            return cuda_failed(__LINE__);
        }
        ++g_launches;
        kp.block_flags = flags;
        kp.unit_counter = unit_counter;
        if (cache == kFlagsFill) flag_cache_filled(a->device, flag_slot, stream);
    }
    kp.out = a->out;
    kp.lse = a->lse;
    kp.o_part = o_part;
    kp.lse_part = lse_part;
    kp.status = dev->status_ptr;
    kp.B = a->batch; kp.H = a->heads; kp.Hk = a->heads_k; kp.Sq = a->seqlen_q; kp.Sk = a->seqlen_k;
    kp.num_splits = plan.num_splits;
    kp.kv_blocks = plan.kv_blocks;
    kp.head_pairs = plan.head_pairs;
    kp.m_pairs = plan.head_pairs ? ceil_div(a->seqlen_q, kBlockM) : ceil_div(a->seqlen_q, 2 * kBlockM);
    kp.dual = plan.dual_split;
    kp.split_groups = plan.dual_split ? ceil_div(plan.num_splits, 2) : plan.num_splits;
    kp.total_units = kp.m_pairs * kp.split_groups * (plan.head_pairs ? a->heads / 2 : a->heads) * a->batch;
    if (plan.unit_cut) {
        uint8_t* slots = static_cast<uint8_t*>(workspace) + plan.workspace_bytes - cut_bytes(plan.grid_x, d);
        // the partials are written with 256-bit stores; a workspace that is only 16-byte
        // aligned keeps every unit whole instead (same grid, every grid-th unit per CTA)
        if ((reinterpret_cast<uintptr_t>(slots) & 31u) == 0) {
            kp.cut_units = plan.unit_cut;
            kp.cut_part = reinterpret_cast<float*>(slots);
            kp.cut_tag = next_cut_tag();
        }
    }
    kp.out_fp32 = a->out_fp32;
    kp.wide_stores = (((reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(o_part)) & 31u) == 0) ? 1 : 0;
    kp.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(d)));
    kp.wait_kcycles = kMaxWaitKcycles;
    kp.mask_bcast = (mask_bs == 0 && a->batch > 1) ? 1 : 0;
    if (rule != nullptr) {
        kp.rule_causal = rule->causal;
        kp.rule_window = rule->window;
        kp.valid_lens = rule->valid_lens;
        if (rule->counter != nullptr) {
            // (a compare-and-swap counter that tolerates any content was measured first: with 148
            // CTAs drawing in waves its retries are quadratic and cost 100 us per launch)
            if (cudaMemsetAsync(rule->counter, 0, sizeof(unsigned int), stream) != cudaSuccess) return cuda_failed(__LINE__);
            kp.unit_counter = rule->counter;
        }
    }
    if (a->disable & FA_SM100_TEST_STALL_MASK) {
        // test only: the mask never arrives, every wait gets a short limit (default 2 M cycles,
        // about a millisecond), the kernel gives up cleanly and reports it
        kp.test_stall_mask = 1;
        const char* env = std::getenv("FA_SM100_TEST_WAIT_KCYCLES");
        const long v = env != nullptr ? std::atol(env) : 0;
        kp.wait_kcycles = v > 0 ? static_cast<unsigned int>(v) : 2000u;
    }

    CUtensorMap tq, tk, tv, tm;
    MapKey key;
    std::memset(&key, 0, sizeof(key));             // padding bytes take part in the compare
    key.q = a->q; key.k = a->k; key.v = a->v; key.mask = mask_ptr;
    key.mask_rs = mask_rs; key.mask_bs = mask_bs;
    key.dtype = a->dtype; key.B = a->batch; key.H = a->heads; key.Hk = a->heads_k;
    key.Sq = a->seqlen_q; key.Sk = a->seqlen_k; key.d = d; key.device = a->device;
    if ((rc = get_maps(key, &tq, &tk, &tv, &tm)) != FA_SM100_OK) return rc;

    const dim3 grid(plan.grid_x, plan.grid_y, plan.grid_z);
    const bool chained = plan.mask_repitched || run_classify;
    const bool bf16 = a->dtype == FA_SM100_BF16;
    const bool list = kp.block_flags != nullptr;
    const int slot = (d == 128 ? 0 : 2) + (bf16 ? 0 : 1) + (list ? 4 : 0) + (rule != nullptr ? 8 : 0);
    if (rule != nullptr) {
        // (a rule launch is a single pass without a skip list: fa_mask_fwd_sm100_rule sees to that)
        if (list || plan.num_splits != 1 || plan.unit_cut != 0 || plan.mask_repitched) return FA_SM100_ERR_SHAPE;
        if (d == 128) rc = bf16 ? launch_fwd<128, true, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                                : launch_fwd<128, false, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
        else rc = bf16 ? launch_fwd<64, true, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                       : launch_fwd<64, false, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
    } else if (d == 128) {
        if (list) rc = bf16 ? launch_fwd<128, true, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                            : launch_fwd<128, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
        else rc = bf16 ? launch_fwd<128, true, false>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                       : launch_fwd<128, false, false>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
    } else {
        if (list) rc = bf16 ? launch_fwd<64, true, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                            : launch_fwd<64, false, true>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
        else rc = bf16 ? launch_fwd<64, true, false>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained)
                       : launch_fwd<64, false, false>(dev, slot, tq, tk, tv, tm, kp, grid, stream, chained);
    }
    if (rc != FA_SM100_OK) return rc;
    if (flag_slot >= 0) flag_cache_read(a->device, flag_slot, stream);
    if (plan.num_splits > 1)
        rc = launch_combine(o_part, lse_part, a->out, a->lse,
                            plan.dual_split ? ceil_div(plan.num_splits, 2) : plan.num_splits, rows, d,
                            a->dtype, a->out_fp32, stream, /*chained=*/true);
    return rc;
}

// ---------------------------------------------------------------------------------
// Built-in scratch for callers that cannot allocate device memory.
// ---------------------------------------------------------------------------------
// The array below is part of the library image: every GPU on which the library is loaded
// carries these FA_SM100_STATIC_SCRATCH_BYTES until the process exits.  Its name is only a
// host-side handle; the device address is looked up once per device with
// cudaGetSymbolAddress and cached.
static __device__ __align__(256) unsigned char g_static_scratch[FA_SM100_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

static int forward_static_scratch(const FaMaskFwdArgs* a, cudaStream_t stream) {
    FaMaskFwdPlan plan;
    int rc = make_plan(a, &plan);
    if (rc != FA_SM100_OK) return rc;
    if (plan.workspace_bytes > FA_SM100_STATIC_SCRATCH_BYTES) return FA_SM100_ERR_WORKSPACE;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        scratch = g_static_scratch_addr[a->device];
        if (scratch == nullptr) {
            // set-up, once per device, with that device current
            DeviceGuard guard(a->device);
            if (guard.err != cudaSuccess) {
                return cuda_failed(__LINE__);
            }
            void* ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
                return cuda_failed(__LINE__);
            }
            g_static_scratch_addr[a->device] = ptr;
            scratch = ptr;
        }
    }
    // (no adaptive pre-pass gating here: that would allocate a pinned host word)
    return forward(a, scratch, FA_SM100_STATIC_SCRATCH_BYTES, stream, /*adaptive_skip=*/false);
}

}  // namespace fa_sm100

// ---------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------
extern "C" {

int fa_mask_fwd_sm100_abi_version(void) { return FA_SM100_ABI_VERSION; }

int fa_mask_fwd_sm100_plan(const FaMaskFwdArgs* args, FaMaskFwdPlan* plan) {
    if (plan == nullptr) return FA_SM100_ERR_NULL;
    return fa_sm100::make_plan(args, plan);
}

int fa_mask_fwd_sm100_workspace_bytes(const FaMaskFwdArgs* args, size_t* bytes) {
    if (bytes == nullptr) return FA_SM100_ERR_NULL;
    FaMaskFwdPlan plan;
    const int rc = fa_sm100::make_plan(args, &plan);
    if (rc != FA_SM100_OK) return rc;
    *bytes = static_cast<size_t>(plan.workspace_bytes);
    return FA_SM100_OK;
}

int fa_mask_fwd_sm100(const FaMaskFwdArgs* args, void* workspace, size_t workspace_bytes,
                      void* stream) {
    return fa_sm100::forward(args, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int fa_mask_fwd_sm100_combine(const float* o_parts, const float* lse_parts, void* out,
                              float* lse_out, int32_t num_parts, int64_t rows, int32_t head_dim,
                              int32_t dtype, int32_t out_fp32, int32_t device, void* stream) {
    if (out == nullptr || (num_parts > 0 && (o_parts == nullptr || lse_parts == nullptr)))
        return FA_SM100_ERR_NULL;
    if (head_dim != 64 && head_dim != 128) return FA_SM100_ERR_HEAD_DIM;
    if (dtype != FA_SM100_FP16 && dtype != FA_SM100_BF16) return FA_SM100_ERR_DTYPE;
    if (num_parts < 0 || num_parts > FA_SM100_MAX_SPLITS) return FA_SM100_ERR_SPLITS;
    if (rows < 0 || device < 0 || device >= fa_sm100::kMaxDevices) return FA_SM100_ERR_SHAPE;
    fa_sm100::DeviceGuard guard(device);
    if (guard.err != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    return fa_sm100::launch_combine(o_parts, lse_parts, out, lse_out, num_parts, rows, head_dim,
                                    dtype, out_fp32, static_cast<cudaStream_t>(stream));
}

int fa_mask_fwd_sm100_combine_packed(const float* packed, int64_t part_stride, void* out, float* lse_out,
                                     int32_t num_parts, int64_t rows, int32_t head_dim, int32_t dtype,
                                     int32_t out_fp32, int32_t device, void* stream) {
    if (out == nullptr || (num_parts > 0 && packed == nullptr)) return FA_SM100_ERR_NULL;
    if (head_dim != 64 && head_dim != 128) return FA_SM100_ERR_HEAD_DIM;
    if (dtype != FA_SM100_FP16 && dtype != FA_SM100_BF16) return FA_SM100_ERR_DTYPE;
    if (num_parts < 0 || num_parts > FA_SM100_MAX_SPLITS) return FA_SM100_ERR_SPLITS;
    if (rows < 0 || device < 0 || device >= fa_sm100::kMaxDevices) return FA_SM100_ERR_SHAPE;
    if (part_stride < rows * (head_dim + 1) || part_stride % 4 != 0) return FA_SM100_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(packed) & 15u) != 0) return FA_SM100_ERR_ALIGN;
    fa_sm100::DeviceGuard guard(device);
    if (guard.err != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    return fa_sm100::launch_combine(packed, packed + rows * head_dim, out, lse_out, num_parts, rows, head_dim,
                                    dtype, out_fp32, static_cast<cudaStream_t>(stream), false, part_stride,
                                    part_stride);
}

int fa_mask_fwd_sm100_combine_peers(const void* part_table, int64_t part_offset, int64_t flag_offset,
                                    int32_t rank, int32_t world, uint32_t seq, void* out, float* lse_out,
                                    int64_t rows, int32_t head_dim, int32_t dtype, int32_t out_fp32,
                                    int32_t device, void* stream) {
    if (out == nullptr || part_table == nullptr) return FA_SM100_ERR_NULL;
    if (head_dim != 64 && head_dim != 128) return FA_SM100_ERR_HEAD_DIM;
    if (dtype != FA_SM100_FP16 && dtype != FA_SM100_BF16) return FA_SM100_ERR_DTYPE;
    if (world < 1 || world > FA_SM100_MAX_SPLITS || rank < 0 || rank >= world) return FA_SM100_ERR_SPLITS;
    if (rows < 0 || seq == 0 || part_offset < 0 || part_offset % 4 != 0 || flag_offset < 0 ||
        device < 0 || device >= fa_sm100::kMaxDevices)
        return FA_SM100_ERR_SHAPE;
    fa_sm100::DeviceGuard guard(device);
    if (guard.err != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    fa_sm100::DeviceInfo* dev = nullptr;
    fa_sm100::query_device(device, &dev);
    int rc = fa_sm100::status_pointer(dev);
    if (rc != FA_SM100_OK) return rc;
    fa_sm100::status_host_setup(dev, static_cast<cudaStream_t>(stream), true);
    if (dev->status_host != nullptr && *static_cast<volatile unsigned int*>(dev->status_host) != 0u)
        return FA_SM100_ERR_DEVICE_WAIT;
    fa_sm100::PeerExchange px;
    px.parts = static_cast<const float* const*>(part_table);
    px.part_offset = part_offset;
    px.flag_offset = flag_offset;
    px.rank = rank;
    px.world = world;
    px.seq = seq;
    px.wait_kcycles = fa_sm100::kMaxWaitKcycles;
    px.status = dev->status_ptr;
    return fa_sm100::launch_combine(nullptr, nullptr, out, lse_out, world, rows, head_dim, dtype, out_fp32,
                                    static_cast<cudaStream_t>(stream), false, 0, 0, &px);
}

int fa_mask_fwd_sm100_device_status(int32_t device, uint32_t* status, int32_t clear) {
    if (status == nullptr) return FA_SM100_ERR_NULL;
    if (device < 0 || device >= fa_sm100::kMaxDevices) return FA_SM100_ERR_SHAPE;
    fa_sm100::DeviceGuard guard(device);
    if (guard.err != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    unsigned int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    if (cudaMemcpyFromSymbol(&v, fa_sm100::g_fa_status, sizeof(v)) != cudaSuccess) {
        return fa_sm100::cuda_failed(__LINE__);
    }
    *status = v;
    if (clear && v != 0) {
        const unsigned int zero = 0;
        if (cudaMemcpyToSymbol(fa_sm100::g_fa_status, &zero, sizeof(zero)) != cudaSuccess) {
            return fa_sm100::cuda_failed(__LINE__);
        }
    }
    if (clear && fa_sm100::g_dev[device].status_host != nullptr)
        *static_cast<volatile unsigned int*>(fa_sm100::g_dev[device].status_host) = 0u;
    return v == 0 ? FA_SM100_OK : FA_SM100_ERR_DEVICE_WAIT;
}

int fa_mask_build_sm100(void* mask, int32_t batch, int32_t seqlen_q, int32_t seqlen_k, int32_t pitch,
                        int32_t dtype, int32_t causal, int32_t window, const int32_t* valid_lens,
                        int32_t device, void* stream) {
    if (mask == nullptr) return FA_SM100_ERR_NULL;
    if (dtype != FA_SM100_FP16 && dtype != FA_SM100_BF16) return FA_SM100_ERR_DTYPE;
    if (batch < 0 || seqlen_q < 0 || seqlen_k < 0 || pitch < seqlen_k || device < 0 ||
        device >= fa_sm100::kMaxDevices)
        return FA_SM100_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(mask) & 1u) != 0) return FA_SM100_ERR_ALIGN;
    const long long rows = static_cast<long long>(batch) * seqlen_q;
    if (rows == 0 || pitch == 0) return FA_SM100_OK;
    if (rows > 0x7fffffffLL) return FA_SM100_ERR_SHAPE;
    fa_sm100::DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return fa_sm100::cuda_failed(__LINE__);
    const unsigned vec_blocks = static_cast<unsigned>((pitch + 8 * 256 - 1) / (8 * 256));
    if (vec_blocks > 65535u) return FA_SM100_ERR_SHAPE;
    const uint32_t neg = dtype == FA_SM100_BF16 ? 0xFF80u : 0xFC00u;
    fa_sm100::fa_mask_build_kernel<<<dim3(static_cast<unsigned>(rows), vec_blocks), 256, 0,
                                     static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t*>(mask), seqlen_q, seqlen_k, pitch, neg, causal, window, valid_lens);
    if (cudaPeekAtLastError() != cudaSuccess) return fa_sm100::cuda_failed(__LINE__);
    ++fa_sm100::g_launches;
    return FA_SM100_OK;
}

int fa_mask_fwd_sm100_rule(const FaMaskFwdArgs* args, int32_t causal, int32_t window, const int32_t* valid_lens,
                           void* workspace, size_t workspace_bytes, void* stream) {
    if (args == nullptr) return FA_SM100_ERR_NULL;
    if (args->struct_size != sizeof(FaMaskFwdArgs)) return FA_SM100_ERR_ABI;
    if (window < 0) return FA_SM100_ERR_SHAPE;
    if (workspace != nullptr && (workspace_bytes < FA_SM100_RULE_WORKSPACE_BYTES ||
                                 (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0))
        return FA_SM100_ERR_WORKSPACE;
    // The same launch as for a mask tensor, as one pass over the keys with whole units and no
    // pre-pass; the mask fields describe a one-plane placeholder that no kernel reads.
    FaMaskFwdArgs a = *args;
    a.mask = a.q;
    a.mask_seqlen_q = a.seqlen_q;
    a.mask_seqlen_k = a.seqlen_k;
    a.mask_row_stride = (static_cast<int64_t>(a.seqlen_k) + 7) & ~static_cast<int64_t>(7);
    a.mask_batch_stride = 0;
    a.num_splits = 1;
    a.out_fp32 = 0;
    a.mask_version = 0;
    a.disable |= FA_SM100_NO_TILE_SKIP | FA_SM100_NO_UNIT_CUT;
    fa_sm100::RuleSpec rule{causal != 0 ? 1 : 0, window, valid_lens, static_cast<unsigned int*>(workspace)};
    return fa_sm100::forward(&a, nullptr, 0, static_cast<cudaStream_t>(stream), true, &rule);
}

int fa_mask_fwd_sm100_static_scratch(const FaMaskFwdArgs* args, void* stream) {
    return fa_sm100::forward_static_scratch(args, static_cast<cudaStream_t>(stream));
}

int fa_mask_fwd_sm100_launch_count(uint64_t* launches) {
    if (launches == nullptr) return FA_SM100_ERR_NULL;
    *launches = fa_sm100::g_launches.load();
    return FA_SM100_OK;
}

const char* fa_mask_fwd_sm100_strerror(int code) {
    switch (code) {
        case FA_SM100_OK: return "ok";
        case FA_SM100_ERR_NULL: return "a required pointer is NULL";
        case FA_SM100_ERR_DTYPE: return "q must be float16 or bfloat16 (k, v, mask must match)";
        case FA_SM100_ERR_SHAPE:
            return "bad shape: sizes must be non-negative, n_heads divisible by n_kv_heads, "
                   "mask (B, 1, >=Sq, >=Sk)";
        case FA_SM100_ERR_HEAD_DIM: return "Only head_dim=64 or head_dim=128 is supported";
        case FA_SM100_ERR_ALIGN: return "q, k, v, out and workspace must be 16-byte aligned";
        case FA_SM100_ERR_WORKSPACE: return "workspace missing or too small";
        case FA_SM100_ERR_ARCH: return "no kernel for this GPU: compute capability 10.x (sm_100a) required";
        case FA_SM100_ERR_CUDA: return "a CUDA call failed";
        case FA_SM100_ERR_SPLITS: return "num_splits out of range";
        case FA_SM100_ERR_DEVICE_WAIT: return "a kernel gave up on a bounded wait (device status word set)";
        case FA_SM100_ERR_ABI: return "FaMaskFwdArgs.struct_size does not match this library";
        default: return "unknown error";
    }
}

}  // extern "C"
