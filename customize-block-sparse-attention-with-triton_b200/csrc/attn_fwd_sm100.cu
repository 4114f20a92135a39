// Forward block-sparse attention for sm_100a.
//
// Persistent kernel: one CTA per SM.  A work item is ONE query block (64 rows) of one (batch, head)
// with its list of key blocks; CTA c starts with item c and then draws further items from an
// optional work counter (or walks a fixed stride).  The list is taken FOUR key tiles at a time
// ("supersteps": tiles a, b, c, d in list order).  The 128 TMEM lanes are split between the
// tiles: lanes 0..63 own tiles a and c, lanes 64..127 own tiles b and d, so that every SM
// sub-partition (32 lanes) has the same amount of exp2 work whatever the sparsity pattern, and a
// softmax warp works through 128 logits per row between two barrier round trips.
//
// The query block sits in shared memory once, between blocks of zero rows: [Z; Q; Z].  The
// 128-row A operand [Q; Z] (Q in rows 0..63) multiplied with [K_a; K_c]^T fills lanes 0..63 of an
// S slot with the logits of tiles a (columns 0..63) and c (columns 64..127) and lanes 64..127 with
// zeros; the operand [Z; Q] with [K_b; K_d]^T then adds the logits of tiles b and d to lanes
// 64..127 (and zeros to the others): eight M=128, N=128, K=16 MMAs per superstep, none of whose
// 128 x 128 outputs is thrown away.
//
// Roles (16 warps); every role walks the same item sequence, so set-up of item i+1 and write-out
// of item i-1 overlap the arithmetic of item i:
//   warp 8      : producer — lists the CTA's first item, then TMA-loads Q and the listed K tiles of
//                 every item into a 2-deep ring of superstages (4 tiles, held until S is
//                 complete), one lane per tile, and tells the lister when to set up the next item
//   warp 14     : lister (also a write-out warp) — draws the next item, lists its key blocks (from
//                 the mask row, or copies the CSR row) into the other list buffer and publishes it
//   warp 15     : V producer — TMA-loads the listed V tiles into a 3-deep ring (held until P V is
//                 complete), one lane per tile.  Only listed tiles are ever loaded.
//   warp 9      : S issuer and TMEM owner
//   warp 10     : P V issuer — O[T] += P_t V_t for the tiles t of the superstep: tiles a, b into the
//                 accumulator of softmax team 0, tiles c, d into that of team 1.  P is read from
//                 TMEM, V is an MN-major shared-memory operand.  The lanes that do not own tile t
//                 hold zeros in t's P columns, so row r of an accumulator only sums products of
//                 the tile owned by lanes 0..63 and row r+64 only of the other one.
//   warps 0..7  : online softmax in two teams of four warps (team = warp / 4, TMEM lane quarter =
//                 warp % 4).  Every warp works on every superstep: team 0 on tiles a, b (columns
//                 0..63 of the slot), team 1 on tiles c, d (columns 64..127); each team has its own
//                 accumulator and (m, l) per lane.  Three S slots (128 TMEM columns) rotate over
//                 the supersteps; a slot is held from the S MMAs until the P V MMAs that read the
//                 probabilities, which overwrite the logits in place, are complete, so while one
//                 slot is with the softmax warps the next already holds its logits and the
//                 previous one is being multiplied with V.  A warp loads its tile's 64 logits,
//                 takes the row maximum, moves the lane's reference maximum if need be (rescaling
//                 its accumulator rows), exponentiates, and stores P (16-bit, 32 columns) over one
//                 half of the tile's columns and zeros over the other half, where the other 64
//                 lanes' P goes: tile t's P ends up in columns [32 t, +32) of the slot.
//   warps 11..14: write-out — merge the four partial results (m, l, O) of every query row (teams x
//                 lanes r / r+64), normalise, store O, LSE and the row maximum.
// TMEM (512 columns): S/P slots 3 x 128, accumulators 2 x 64.
//
// Numerics follow the reference's loop (fa2_custom_mask/fa2_fwd.py:150-196): logits scaled by
// sm_scale*log2(e), exp2 domain, fp32 row sums of the fp32 probabilities, P rounded to the input
// dtype before P V.  The running maximum is only advanced when it grew by more than 8 (a factor
// 256), which leaves O = acc / l unchanged because both use the same reference maximum.  Which
// partial result a tile goes into depends on its position in the row's list alone, so results do
// not depend on which CTA computes an item.
//
// Every wait is bounded; a wait that gives up raises a CTA-wide flag, every role then falls
// through its loops without touching barriers' data again, and TMEM is always released.  Every
// barrier is waited on only by warps that see each of its phases, or that know the barrier to be
// at most one phase behind (a parity wait cannot tell a phase from the one two before it).
#include <math.h>
#include <string.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace bsa {

constexpr int kKStages = 2;     // K superstages (4 tiles) in flight: held from load to S complete
constexpr int kVStages = 3;     // V superstages (4 tiles) in flight: held from load to P V complete
constexpr int kSlots = 3;       // S/P slots (128 TMEM columns): held from S issue to P V complete
constexpr int kFwdThreads = 512;
constexpr int kSoftmaxWarps = 8, kProducerWarp = 8, kSWarp = 9, kPvWarp = 10;  // warps 11..14 write out
constexpr int kVProducerWarp = 15;  // = the last warp
constexpr int kListerWarp = 14;     // the write-out warp that also sets up the items
constexpr int kGoBefore = 2;         // ordered hand-out: K superstages before an item's end at which the next is drawn
constexpr uint32_t kTileBytes = 64 * 64 * 2;       // one Q, K or V tile
constexpr uint32_t kFwdTmemCols = 512;
// TMEM columns: slot r at 128 r; accumulator of softmax team T at 384 + 64 T.
constexpr uint32_t kTmemO = 384;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kFwdMaxTiles = 2048;  // key blocks per row that a CTA can list (N <= 131072)
constexpr int kMaxSorted = 320;     // items beyond the first round that a CTA can put in order
constexpr uint16_t kColPartial = 0x8000;  // list entry in shared memory: the tile has masked elements
constexpr uint16_t kColIndex = 0x7fff;

struct FwdSmem {
  uint8_t qz[5][kTileBytes];                  // Z, Q (even items), Z, Q (odd items), Z
  uint8_t k[kKStages][4][kTileBytes];         // tiles in the order a, c, b, d
  uint8_t v[kVStages][4][kTileBytes];         // tiles in the order a, b, c, d
  float xfer[32][65];                         // write-out: lanes 64..127 hand over, [col][row]
  uint16_t cols[2][kFwdMaxTiles];             // by item parity: the item's key-block list (| kColPartial)
  alignas(16) int cnt[kMaxSorted];            // sort keys (tile count, item) of the items beyond the first round
  int order[kMaxSorted];                      // those items, longest first
  int ntiles[2];
  int item[2];                                // by item parity: the work item, -1 = no more work
  float mref[2][2][128];                      // by item parity, softmax team, lane
  float lsum[2][2][128];
  float mtrue[2][2][128];
  uint64_t order_full;                        // `order` is ready
  uint64_t list_full[2];                      // lister -> everyone: list and tile count ready
  uint64_t setup_go[2];                       // producer -> lister: time to set up the next item
  uint64_t q_full[2], q_free[2];
  uint64_t k_full[kKStages];
  uint64_t k_empty[kKStages];                 // S of the superstep complete
  uint64_t v_full[kVStages];
  uint64_t v_empty[kVStages];                 // P V of the superstep complete
  uint64_t s_full[kSlots];                    // S of the superstep complete
  uint64_t p_full[kSlots][2];                 // by team: its four warps stored P of the superstep
  uint64_t pv_done[kSlots];                   // P V of the superstep complete: slot free, O current
  uint64_t o_full[2];                         // last P V of the item done
  uint64_t stats_full[2];                     // softmax warps published (m, l) of the item
  uint64_t o_free[2];                         // write-out holds accumulators/stats/header in registers
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(FwdSmem) + 1024 <= 232448, "FwdSmem exceeds the shared memory of one CTA");

struct FwdParams {
  const int32_t* row_ptr;   // list mode: CSR row lists
  const int32_t* col_idx;
  const uint8_t* block;     // mask mode (block != nullptr): the kernel lists the mask rows itself
  int64_t ms0, ms1, ms2, ms3;
  const uint8_t* dense;     // optional element-level mask for the tiles marked partial
  int64_t ds0, ds1, ds2;
  void* o;
  int64_t o_sb, o_sh, o_sn;
  float* lse2;
  float* rowmax;
  int B, H, N, nb;
  int row_begin, nrows;     // the query-block rows [row_begin, row_begin + nrows) of every head
  int list_b_stride, list_h_stride;
  int items;                // B * H * nrows
  float scale_log2;
  int32_t* status;
  int32_t* ticket;          // optional work counter (0 at kernel start, left 0): dynamic item hand-out
  int wide_stores;          // rows of O start on 32-byte boundaries
};

enum FwdFail : int { kFailProducer = 1, kFailMma = 2, kFailSoftmax = 3, kFailOut = 4 };

__device__ __forceinline__ void fwd_give_up(FwdSmem* sm, int32_t* status, int code) {
  sm->abort_flag = 1;
  report_status(status, code);
}

// exp2 of one 32-column chunk of S against the row's reference maximum; returns the packed
// 16-bit probabilities and adds their fp32 sum to l.  The scale-and-subtract and the running sums
// take two columns per instruction.
template <bool kBf16>
__device__ __forceinline__ void exp_chunk(const uint32_t* sr, float c, float neg_m, uint32_t* pk,
                                          float& l) {
  const uint64_t c2 = pack_f32x2(c, c), m2 = pack_f32x2(neg_m, neg_m);
  uint64_t l01 = pack_f32x2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    float z0, z1, z2, z3;
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), c2, m2),
                 z0, z1);
    unpack_f32x2(
        fma_f32x2(pack_f32x2(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])), c2, m2), z2,
        z3);
    const float p0 = ex2_approx(z0), p1 = ex2_approx(z1), p2 = ex2_approx(z2), p3 = ex2_approx(z3);
    l01 = add_f32x2(add_f32x2(l01, pack_f32x2(p0, p1)), pack_f32x2(p2, p3));
    pk[i / 2] = pack_2x16<kBf16>(p0, p1);
    pk[i / 2 + 1] = pack_2x16<kBf16>(p2, p3);
  }
  float a0, a1;
  unpack_f32x2(l01, a0, a1);
  l += a0 + a1;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));  // one instruction on sm_100
  return d;
}

__device__ __forceinline__ float max_chunk(const uint32_t* sr) {
  float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]);
#pragma unroll
  for (int i = 2; i < 30; i += 4) {
    mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
    mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
  }
  return max3(mx0, mx1, fmaxf(__uint_as_float(sr[30]), __uint_as_float(sr[31])));
}

// Work item w -> (batch, head, query block); late (long, if causal) query blocks of a head first.
struct FwdItem {
  int b, h, mb;
};
__device__ __forceinline__ FwdItem fwd_item(int w, const FwdParams& p) {
  const int bh = w / p.nrows;
  FwdItem it;
  it.mb = p.row_begin + p.nrows - 1 - (w - bh * p.nrows);
  it.b = bh / p.H;
  it.h = bh - it.b * p.H;
  return it;
}

// Mask row of a work item (mask mode); list_*_stride are 0 for a broadcast axis and 1 otherwise.
__device__ __forceinline__ const uint8_t* fwd_mask_row(const FwdItem& it, const FwdParams& p) {
  return p.block + (it.b * p.list_b_stride) * p.ms0 + (it.h * p.list_h_stride) * p.ms1 +
         static_cast<int64_t>(it.mb) * p.ms2;
}

// Number of kept blocks in a contiguous mask row of nb bytes, read by ONE thread: bytes up to the
// first 4-byte boundary, then words (a word's non-zero bytes are counted with a byte-wise
// compare), then the tail.
__device__ __forceinline__ int fwd_count_row(const uint8_t* row, int nb) {
  int n = 0, c = 0;
  const int head = static_cast<int>((4u - (reinterpret_cast<uintptr_t>(row) & 3u)) & 3u);
  for (; c < head && c < nb; ++c) n += __ldg(row + c) != 0 ? 1 : 0;
  const uint32_t* w = reinterpret_cast<const uint32_t*>(row + c);
  const int words = (nb - c) >> 2;
  int k = 0;
  for (; k + 16 <= words; k += 16) {
    uint32_t a[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) a[j] = __ldg(w + k + j);
    int bits = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) bits += __popc(__vcmpne4(a[j], 0u));
    n += bits >> 3;
  }
  for (; k + 4 <= words; k += 4) {
    const uint32_t a0 = __ldg(w + k), a1 = __ldg(w + k + 1), a2 = __ldg(w + k + 2),
                   a3 = __ldg(w + k + 3);
    n += (__popc(__vcmpne4(a0, 0u)) + __popc(__vcmpne4(a1, 0u)) + __popc(__vcmpne4(a2, 0u)) +
          __popc(__vcmpne4(a3, 0u))) >> 3;
  }
  for (; k < words; ++k) n += __popc(__vcmpne4(__ldg(w + k), 0u)) >> 3;
  for (c += 4 * words; c < nb; ++c) n += __ldg(row + c) != 0 ? 1 : 0;
  return n;
}

// When the items are handed out through the work counter and there are at most a few per CTA, it
// matters who gets which: rows of a random mask differ in length, and the kernel is as slow as
// the CTA with the largest sum.  The first round is fixed (CTA c takes item c); the remaining
// items are handed out longest first, so that the CTAs that finish their first item early take
// the long ones.  Every CTA works the order out for itself (same input, same result) with the
// four write-out warps, which have nothing to do during the first item: one thread per row counts
// the row's kept blocks, then every thread ranks its row among all.
__device__ __forceinline__ void fwd_build_order(FwdSmem* sm, const FwdParams& p, int tid, int first,
                                                int n2) {
  for (int j = tid; j < n2; j += 128) {
    const FwdItem it = fwd_item(first + j, p);
    int n;
    if (p.block != nullptr) {
      n = fwd_count_row(fwd_mask_row(it, p), p.nb);
    } else {
      const int64_t li =
          static_cast<int64_t>(it.b * p.list_b_stride + it.h * p.list_h_stride) * p.nb + it.mb;
      n = __ldg(p.row_ptr + li + 1) - __ldg(p.row_ptr + li);
    }
    // one key per item, all different: longer rows first, equal rows in item order
    sm->cnt[j] = n * 512 + (511 - j);
  }
  const int n4 = (n2 + 3) & ~3;
  for (int j = n2 + tid; j < n4; j += 128) sm->cnt[j] = -1;  // padding ranks behind every item
  named_barrier_sync(2, 128);
  for (int j = tid; j < n2; j += 128) {
    const int kj = sm->cnt[j];
    int r0 = 0, r1 = 0, r2 = 0, r3 = 0;
    for (int k = 0; k < n4; k += 4) {
      const int4 c = *reinterpret_cast<const int4*>(&sm->cnt[k]);
      r0 += c.x > kj ? 1 : 0;
      r1 += c.y > kj ? 1 : 0;
      r2 += c.z > kj ? 1 : 0;
      r3 += c.w > kj ? 1 : 0;
    }
    sm->order[(r0 + r1) + (r2 + r3)] = j;
  }
  named_barrier_sync(2, 128);
  if (tid == 0) mbar_arrive(smem_u32(&sm->order_full));
}

// Lists the key blocks of work item w into the list buffer of parity par (one warp) and publishes
// list, tile count and item.
template <bool kElementMask>
__device__ __forceinline__ void fwd_list_item(FwdSmem* sm, const FwdParams& p, int w, int par,
                                              int lane) {
  const FwdItem it = fwd_item(w, p);
  uint16_t* cols = sm->cols[par];
  int n_tiles = 0;
  if (p.block != nullptr) {
    // mask mode: ordered compaction of the kept blocks of mask row (b, h, mb)
    const uint8_t* mrow = fwd_mask_row(it, p);
    // 128 columns per pass, four independent loads per lane; the next pass's loads are issued
    // before this pass's ballots, so a row costs one round trip to L2 rather than one per pass
    int byte[4], next[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int c = 32 * jj + lane;
      next[jj] = c < p.nb ? mrow[c * p.ms3] : 0;
    }
    for (int c0 = 0; c0 < p.nb; c0 += 128) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        byte[jj] = next[jj];
        const int c = c0 + 128 + 32 * jj + lane;
        next[jj] = c < p.nb ? mrow[c * p.ms3] : 0;
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const unsigned bal = __ballot_sync(0xffffffffu, byte[jj] != 0);
        if (byte[jj] != 0)
          cols[n_tiles + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(
              (c0 + 32 * jj + lane) | (kElementMask && byte[jj] == 2 ? kColPartial : 0));
        n_tiles += __popc(bal);
      }
    }
  } else {
    const int64_t li =
        static_cast<int64_t>(it.b * p.list_b_stride + it.h * p.list_h_stride) * p.nb + it.mb;
    const int beg = __ldg(p.row_ptr + li);
    n_tiles = __ldg(p.row_ptr + li + 1) - beg;
    for (int jj = lane; jj < n_tiles; jj += 32) {
      const int e = __ldg(p.col_idx + beg + jj);
      cols[jj] = static_cast<uint16_t>(
          (e & kColIndex) | (kElementMask && (e & BSA_LIST_PARTIAL_FLAG) ? kColPartial : 0));
    }
  }
  __syncwarp();
  if (lane == 0) {
    sm->ntiles[par] = n_tiles;
    sm->item[par] = w;
    mbar_arrive(smem_u32(&sm->list_full[par]));  // release: count and list are visible
  }
}

// kElementMask: the instantiation that applies a dense mask inside the tiles marked partial; the
// plain one carries none of that code.
template <bool kBf16, bool kElementMask>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;
  const int stride = gridDim.x;
  // items beyond the first round; few enough per CTA for their order to matter?  (mask mode
  // needs contiguous mask rows for the count)
  const int n2 = p.items - stride;
  const bool sorted = p.ticket != nullptr && n2 > 1 && n2 <= kMaxSorted &&
                      (p.block == nullptr || p.ms3 == 1);

  // ---- set-up ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm->list_full[i]), 1);
      mbar_init(smem_u32(&sm->setup_go[i]), 1);
      mbar_init(smem_u32(&sm->q_full[i]), 1);
      mbar_init(smem_u32(&sm->q_free[i]), 1);
      mbar_init(smem_u32(&sm->o_full[i]), 1);
      mbar_init(smem_u32(&sm->stats_full[i]), kSoftmaxWarps);
      mbar_init(smem_u32(&sm->o_free[i]), 4);  // one arrival per write-out warp
    }
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(smem_u32(&sm->k_full[s]), 1);
      mbar_init(smem_u32(&sm->k_empty[s]), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(smem_u32(&sm->v_full[s]), 1);
      mbar_init(smem_u32(&sm->v_empty[s]), 1);
    }
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(smem_u32(&sm->s_full[s]), 1);
      mbar_init(smem_u32(&sm->p_full[s][0]), kSoftmaxWarps / 2);
      mbar_init(smem_u32(&sm->p_full[s][1]), kSoftmaxWarps / 2);
      mbar_init(smem_u32(&sm->pv_done[s]), 1);
    }
    mbar_init(smem_u32(&sm->order_full), 1);
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  {
    // the three blocks of zero rows around the two query buffers; the MMAs read them through the
    // async proxy
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    constexpr int kVecs = kTileBytes / 16;
    for (int i = threadIdx.x; i < 3 * kVecs; i += kFwdThreads)
      reinterpret_cast<uint4*>(sm->qz[2 * (i / kVecs)])[i % kVecs] = z;
    fence_proxy_async_smem();
  }
  if (warp == kSWarp) {
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->abort_flag;

  if (warp == kProducerWarp) {
    // =========================== producer ===========================
    bool ok = true;
    // Loads Q and the K tiles of the listed key blocks from the list the lister published, and
    // tells the lister when to set up the next item.  A set-up takes 3-4 thousand cycles (the draw
    // from the work counter, the mask row, the ballots in a warp that shares its scheduler with
    // two softmax warps), about two supersteps.  With many items per CTA it is started as soon as
    // an item begins; with the few items of the ordered hand-out, where it matters that a CTA
    // draws its next item only when it is about to need it, kGoBefore superstages before the end.
    int gs = 0;  // supersteps issued so far by this CTA (ring position)
    int qi = 0;  // non-empty items so far (Q buffer position)
    fwd_list_item<kElementMask>(sm, p, blockIdx.x, 0, lane);  // the CTA's own first item
    for (int i = 0; ok; ++i) {
      const int par = i & 1;
      ok = mbar_wait_warp(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      const int w = *const_cast<volatile int*>(&sm->item[par]);
      if (w < 0) break;  // no more work
      const FwdItem it = fwd_item(w, p);
      const int n_tiles = *const_cast<volatile int*>(&sm->ntiles[par]);
      const uint16_t* cols = sm->cols[par];
      const int n_super = (n_tiles + 3) >> 2;
      if (n_super > 0) {
        const int qpar = qi & 1;
        if (qi >= 2) ok = mbar_wait_warp(smem_u32(&sm->q_free[qpar]), ((qi - 2) >> 1) & 1, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t bar = smem_u32(&sm->q_full[qpar]);
          mbar_expect_tx(bar, kTileBytes);
          tma_load_4d(smem_u32(sm->qz[1 + 2 * qpar]), &tm_q, bar, 0, it.mb * 64, it.h, it.b);
        }
        ++qi;
      }
      const int u_go = sorted ? max(n_super - kGoBefore, 0) : 0;
      if (n_super == 0 && lane == 0) mbar_arrive(smem_u32(&sm->setup_go[par]));
      // One lane per tile issues its load: a single thread can start a tile load only every couple
      // of hundred cycles, which four loads in a row would turn into the kernel's bound.
      for (int u = 0; u < n_super; ++u) {
        if (u == u_go && lane == 0) mbar_arrive(smem_u32(&sm->setup_go[par]));
        const int g = gs + u, ks = g % kKStages;
        const int nt = min(4, n_tiles - 4 * u);
        ok = mbar_wait_warp(smem_u32(&sm->k_empty[ks]), ((g / kKStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        const uint32_t bar = smem_u32(&sm->k_full[ks]);
        if (lane == 0) mbar_expect_tx(bar, kTileBytes * nt);
        __syncwarp();
        if (lane < nt)  // shared-memory order a, c, b, d
          tma_load_4d(smem_u32(sm->k[ks][((lane & 1) << 1) | (lane >> 1)]), &tm_k, bar, 0,
                      static_cast<int>(cols[4 * u + lane] & kColIndex) * 64, it.h, it.b);
      }
      gs += n_super;
    }
    if (!ok) fwd_give_up(sm, p.status, kFailProducer);
  } else if (warp == kVProducerWarp) {
    // =========================== V producer ===========================
    // Loads the V tiles of the listed key blocks, one lane per tile, from the list the producer
    // published; a warp of its own, so that waiting for a free V stage (P V complete) never holds
    // back the K tiles of a later superstep.
    bool ok = true;
    int gs = 0;
    for (int i = 0; ok; ++i) {
      const int par = i & 1;
      ok = mbar_wait_warp(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      const int w = *const_cast<volatile int*>(&sm->item[par]);
      if (w < 0) break;  // no more work
      const FwdItem it = fwd_item(w, p);
      const int n_tiles = *const_cast<volatile int*>(&sm->ntiles[par]);
      const int n_super = (n_tiles + 3) >> 2;
      const uint16_t* cols = sm->cols[par];
      for (int u = 0; u < n_super; ++u, ++gs) {
        const int vs = gs % kVStages;
        const int nt = min(4, n_tiles - 4 * u);
        ok = mbar_wait_warp(smem_u32(&sm->v_empty[vs]), ((gs / kVStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        const uint32_t bar = smem_u32(&sm->v_full[vs]);
        if (lane == 0) mbar_expect_tx(bar, kTileBytes * nt);
        __syncwarp();
        if (lane < nt)
          tma_load_4d(smem_u32(sm->v[vs][lane]), &tm_v, bar, 0,
                      static_cast<int>(cols[4 * u + lane] & kColIndex) * 64, it.h, it.b);
      }
    }
    if (!ok) fwd_give_up(sm, p.status, kFailProducer);
  } else if (warp == kSWarp) {
    // =========================== S issuer ===========================
    constexpr uint32_t idesc_n128 = umma_idesc(kBf16, 0, 0, 128, 128);
    constexpr uint32_t idesc_n64 = umma_idesc(kBf16, 0, 0, 128, 64);
    const bool leader = elect_one();
    const uint64_t desc_qz = smem_desc_sw128(smem_u32(sm->qz[0]), 16, 1024);
    const uint64_t desc_k0 = smem_desc_sw128(smem_u32(sm->k[0][0]), 16, 1024);
    constexpr uint64_t kTileDesc = kTileBytes >> 4;  // one tile further, in descriptor units
    bool ok = true;
    int gs = 0, qi = 0;
    for (int i = 0; ok; ++i) {
      const int par = i & 1;
      ok = mbar_wait_warp(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      if (*const_cast<volatile int*>(&sm->item[par]) < 0) break;  // no more work
      const int n_tiles = *const_cast<volatile int*>(&sm->ntiles[par]);
      const int n_super = (n_tiles + 3) >> 2;
      if (n_super == 0) continue;
      const int qpar = qi & 1;
      ok = mbar_wait_warp(smem_u32(&sm->q_full[qpar]), (qi >> 1) & 1, abort_flag);
      if (!ok) break;
      // [Z; Q] starts at the zero block in front of the query buffer, [Q; Z] at the buffer itself
      const uint64_t desc_bot = desc_qz + static_cast<uint64_t>(2 * qpar) * kTileDesc;
      const uint64_t desc_top = desc_bot + kTileDesc;
      for (int u = 0; u < n_super; ++u, ++gs) {
        const int ks = gs % kKStages, slot = gs % kSlots;
        const int nt = min(4, n_tiles - 4 * u);
        ok = mbar_wait_warp(smem_u32(&sm->k_full[ks]), (gs / kKStages) & 1, abort_flag);
        if (!ok) break;
        // the slot's previous user, three supersteps ago, must have had its P V completed
        if (gs >= kSlots)
          ok = mbar_wait_warp(smem_u32(&sm->pv_done[slot]), ((gs - kSlots) / kSlots) & 1,
                              abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          const uint32_t d = tmem + 128 * slot;
          const uint64_t desc_ac = desc_k0 + static_cast<uint64_t>(ks * 4) * kTileDesc;
          const uint64_t desc_bd = desc_ac + 2 * kTileDesc;
          const uint32_t id_ac = nt >= 3 ? idesc_n128 : idesc_n64;
          const uint32_t id_bd = nt >= 4 ? idesc_n128 : idesc_n64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_ss(d, desc_top + 2 * kk, desc_ac + 2 * kk, id_ac, kk > 0);
          if (nt >= 2) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_ss(d, desc_bot + 2 * kk, desc_bd + 2 * kk, id_bd, 1);
          }
          tc_commit(smem_u32(&sm->s_full[slot]));
          tc_commit(smem_u32(&sm->k_empty[ks]));
          if (u == n_super - 1) tc_commit(smem_u32(&sm->q_free[qpar]));  // Q buffer reusable
        }
      }
      ++qi;
    }
    if (!ok) fwd_give_up(sm, p.status, kFailMma);
  } else if (warp == kPvWarp) {
    // =========================== P V issuer ===========================
    constexpr uint32_t idesc_pv = umma_idesc(kBf16, 0, 1, 128, 64);  // P (TMEM) x V (MN-major)
    const bool leader = elect_one();
    const uint64_t desc_v0 = smem_desc_sw128(smem_u32(sm->v[0][0]), 8192, 1024);
    bool ok = true;
    int gs = 0;
    for (int i = 0; ok; ++i) {
      const int par = i & 1;
      ok = mbar_wait_warp(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      if (*const_cast<volatile int*>(&sm->item[par]) < 0) break;  // no more work
      const int n_tiles = *const_cast<volatile int*>(&sm->ntiles[par]);
      const int n_super = (n_tiles + 3) >> 2;
      // the accumulators are free once the previous item has been written out; the softmax warps
      // meanwhile work ahead
      if (i >= 1)
        ok = mbar_wait_warp(smem_u32(&sm->o_free[par ^ 1]), ((i - 1) >> 1) & 1, abort_flag);
      if (!ok) break;
      if (n_super == 0) {
        if (leader) mbar_arrive(smem_u32(&sm->o_full[par]));
        continue;
      }
      for (int u = 0; u < n_super; ++u, ++gs) {
        const int vs = gs % kVStages, slot = gs % kSlots;
        const int nt = min(4, n_tiles - 4 * u);
        ok = mbar_wait_warp(smem_u32(&sm->v_full[vs]), (gs / kVStages) & 1, abort_flag);
        if (!ok) break;
        // Tiles a, b go to the accumulator of team 0 as soon as that team has stored their P, tiles
        // c, d to that of team 1; the first product of an item into an accumulator starts it
        // afresh.  Keys [16 kk, +16) of tile t sit at column 32 t + 8 kk of the slot; the lanes
        // that do not own the tile hold zeros there.
        const uint32_t p_slot = tmem + 128 * slot;
        for (int team = 0; team < 2 && ok; ++team) {
          ok = mbar_wait_warp(smem_u32(&sm->p_full[slot][team]), (gs / kSlots) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          if (leader) {
            const uint32_t o_acc = tmem + kTmemO + 64 * team;
            for (int t = 2 * team; t < min(nt, 2 * team + 2); ++t) {
              const uint64_t desc_v = desc_v0 + static_cast<uint64_t>((vs * 4 + t) * (kTileBytes >> 4));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ts(o_acc, p_slot + 32 * t + 8 * kk, desc_v + 128 * kk, idesc_pv,
                        (u > 0) || (t & 1) || (kk > 0));
            }
          }
        }
        if (!ok) break;
        if (leader) {
          tc_commit(smem_u32(&sm->v_empty[vs]));
          tc_commit(smem_u32(&sm->pv_done[slot]));
          if (u == n_super - 1) tc_commit(smem_u32(&sm->o_full[par]));
        }
      }
    }
    if (!ok) fwd_give_up(sm, p.status, kFailMma);
  } else if (warp < kSoftmaxWarps) {
    // =========================== softmax ===========================
    const int team = warp >> 2;       // team 0 takes tiles a, b of every superstep, team 1 tiles c, d
    const int quarter = warp & 3;     // TMEM lane quarter this warp may touch
    const int half = quarter >> 1;    // lanes 0..63 own tiles a, c of a superstep, 64..127 b, d
    const int t_mine = 2 * team + half, t_other = 2 * team + (half ^ 1);
    const int lane_row = quarter * 32 + lane;  // TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem + lane_base + kTmemO + 64 * team;
    // columns of a slot: the team's logits at [64 team, +64); this warp's P over the first or the
    // second half of them, zeros over the other half (where the other lanes' P goes)
    const uint32_t col_s = 64u * team;
    const uint32_t col_p = col_s + 32u * half, col_z = col_s + 32u * (half ^ 1);
    const float c = p.scale_log2;
    bool ok = true;
    int g0 = 0;  // supersteps of all earlier items of this CTA
    for (int i = 0; ok; ++i) {
      const int par = i & 1;
      ok = mbar_wait_warp(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      const int w_item = *const_cast<volatile int*>(&sm->item[par]);
      if (w_item < 0) break;  // no more work
      const int n_tiles = *const_cast<volatile int*>(&sm->ntiles[par]);
      const int n_super = (n_tiles + 3) >> 2;
      const uint16_t* cols = sm->cols[par];
      float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
      bool next_ready = false;  // the S barrier of the coming superstep has been seen complete
      // this lane's row of the element-level mask, if there is one
      const uint8_t* mask_row = nullptr;
      if constexpr (kElementMask) {
        const FwdItem it = fwd_item(w_item, p);
        mask_row = p.dense + it.b * p.ds0 + it.h * p.ds1 +
                   static_cast<int64_t>(it.mb * 64 + (quarter & 1) * 32 + lane) * p.ds2;
      }

      for (int u = 0; u < n_super; ++u) {
        const int g = g0 + u;
        const int slot = g % kSlots;
        const uint32_t s_addr = tmem + lane_base + 128 * slot;
        const int nt = min(4, n_tiles - 4 * u);
        // A tile with masked elements inside: fetch this row's 64 mask bytes while S is on its way
        uint16_t entry = 0;
        if constexpr (kElementMask) entry = t_mine < nt ? cols[4 * u + t_mine] : 0;
        const bool partial = kElementMask && (entry & kColPartial) != 0;  // warp-uniform
        uint4 mw[4];
        if (partial) {
          const uint4* mp = reinterpret_cast<const uint4*>(mask_row + (entry & kColIndex) * 64);
#pragma unroll
          for (int j = 0; j < 4; ++j) mw[j] = __ldg(mp + j);
        }
        if (!next_ready) {
          ok = mbar_wait_warp(smem_u32(&sm->s_full[slot]), (g / kSlots) & 1, abort_flag);
          if (!ok) break;
        }
        tc_fence_after();
        if (t_mine < nt) {
          uint32_t sr[64];
          tmem_ld_32x32b_x32(s_addr + col_s, sr);
          tmem_ld_32x32b_x32(s_addr + col_s + 32, sr + 32);
          tc_wait_ld();
          // the other lanes' tile of this team reads these lanes too: zeros (the logits are in
          // registers now); stored first, so that it drains under the arithmetic
          if (t_other < nt) tmem_st_zero_32x32b_x32(s_addr + col_z);
          if (partial) {
            // masked elements become -inf: they take no part in the maximum and exponentiate to 0
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w4[4] = {mw[j].x, mw[j].y, mw[j].z, mw[j].w};
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint32_t nz = __vcmpne4(w4[q4], 0u);  // 0xff in every byte that keeps its element
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                  const uint32_t keep = __byte_perm(nz, 0u, 0x1111u * bb);
                  const int i = 16 * j + 4 * q4 + bb;
                  sr[i] = (sr[i] & keep) | (0xff800000u & ~keep);
                }
              }
            }
          }
          const float zmax = fmaxf(max_chunk(sr), max_chunk(sr + 32)) * c;
          m_true = fmaxf(m_true, zmax);
          float alpha = 1.f;
          bool rescale = false;
          if (m_ref == -INFINITY) {
            m_ref = zmax;  // first tile of this lane in this item: O and l are still zero
          } else if (zmax > m_ref + kRescaleThreshold) {
            alpha = ex2_approx(m_ref - zmax);
            l *= alpha;
            m_ref = zmax;
            rescale = true;
          }
          if (__any_sync(0xffffffffu, rescale)) {
            // this warp's O rows must hold the team's previous product (the superstep before) first
            ok = mbar_wait_warp(smem_u32(&sm->pv_done[(g - 1) % kSlots]), ((g - 1) / kSlots) & 1,
                                abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int part = 0; part < 4; ++part) {
              uint32_t orow[16];
              tmem_ld_32x32b_x16(o_addr + 16 * part, orow);
              tc_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j)
                orow[j] = __float_as_uint(__uint_as_float(orow[j]) * alpha);
              tmem_st_32x32b_x16(o_addr + 16 * part, orow);
            }
          }
          // (a row with nothing kept so far has m_ref = -inf: its logits are all -inf, and with a
          // zero in place of the maximum they exponentiate to 0 instead of NaN)
          const float neg_m = (kElementMask && m_ref == -INFINITY) ? 0.f : -m_ref;
          uint32_t pk[16];
          exp_chunk<kBf16>(sr, c, neg_m, pk, l);
          tmem_st_32x32b_x16(s_addr + col_p, pk);
          exp_chunk<kBf16>(sr + 32, c, neg_m, pk, l);
          tmem_st_32x32b_x16(s_addr + col_p + 16, pk);
        } else if (t_other < nt) {
          tmem_st_zero_32x32b_x32(s_addr + col_z);
        }
        // Look at the next superstep's S barrier now: the round trip to it runs under the drain of
        // the stores, and if S is there (it normally is: three slots) the wait at the top of the
        // loop is skipped.
        bool polled = false;
        if (u + 1 < n_super)
          polled = mbar_test(smem_u32(&sm->s_full[(g + 1) % kSlots]), ((g + 1) / kSlots) & 1);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[slot][team]));
        next_ready = __all_sync(0xffffffffu, polled);
      }
      if (!ok) break;

      // publish this item's (m, l) of the warp's lanes; the slots of item i-2 must have been read
      if (i >= 2) ok = mbar_wait_warp(smem_u32(&sm->o_free[par]), ((i - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      sm->mref[par][team][lane_row] = m_ref;
      sm->lsum[par][team][lane_row] = l;
      sm->mtrue[par][team][lane_row] = m_true;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->stats_full[par]));
      g0 += n_super;
    }
    if (!ok) fwd_give_up(sm, p.status, kFailSoftmax);
  } else {
    // =========================== write-out ===========================
    // Merges the four partial results of every query row (teams 0 / 1 x lanes r / r+64).
    // A warp reads both accumulators of its own lanes from TMEM; lanes 64..127 hand their weighted
    // rows to lanes 0..63 through shared memory, 32 columns at a time.  All named barriers of an
    // iteration are always executed, also after a give-up, and the last one carries the give-up
    // vote, so that no warp of this role can be left waiting at one.
    //
    // One of the four warps is also the lister: it sets up item i+1 when the producer says so
    // during item i, i.e. between its write-outs of items i-1 and i (the producer lists the
    // CTA's first item itself, which nothing can overlap).  The draw
    // from the work counter, the mask row and the ballots take a couple of thousand cycles, which
    // in the producer's own instruction stream held back the K tiles of the current item.
    const int quarter = warp & 3;  // lane quarter a warp may touch = its index mod 4
    const bool lister = warp == kListerWarp;
    bool ok = true;
    bool terminal = p.ticket == nullptr;  // drew a ticket past the end (or draws none)
    int lw = blockIdx.x;
    // Lister (one of the four warps): draws item j >= 1, lists its key blocks into the list buffer
    // of j's parity and publishes them, or publishes that there is no further item.  A wait that
    // gives up leaves ok = false and nothing published.
    auto set_up = [&](int j) {
      const int par = j & 1;
      {
        // next item: the following ticket when items are handed out dynamically, else a fixed stride
        if (p.ticket != nullptr) {
          int t = 0;
          if (lane == 0) {
            t = atomicAdd(p.ticket, 1);
            // every CTA draws until its first ticket past the end, so the launch draws exactly
            // `items` tickets in all; whoever draws the last one leaves the counter at zero
            if (t == p.items - 1) atomicExch(p.ticket, 0);
          }
          t = __shfl_sync(0xffffffffu, t, 0);
          terminal = t >= n2;
          if (sorted && t < n2) {
            if (j == 1) ok = mbar_wait_warp(smem_u32(&sm->order_full), 0, abort_flag);
            if (!ok) return;
            t = *const_cast<volatile int*>(&sm->order[t]);
          }
          lw = stride + t;
        } else {
          lw += stride;
        }
      }
      // the list buffer (and the tile count) of item j-2 must have been read by everyone
      if (j >= 2)
        ok = mbar_wait_warp_idle(smem_u32(&sm->o_free[par]), ((j - 2) >> 1) & 1, abort_flag, 128);
      if (!ok) return;
      if (lw >= p.items) {
        if (lane == 0) {
          sm->item[par] = -1;
          mbar_arrive(smem_u32(&sm->list_full[par]));
        }
        return;
      }
      fwd_list_item<kElementMask>(sm, p, lw, par, lane);
    };

    if (sorted) fwd_build_order(sm, p, quarter * 32 + lane, stride, n2);
    const int half = quarter >> 1;
    const int lane_row = quarter * 32 + lane;
    const int r_blk = (quarter & 1) * 32 + lane;  // row of the query block
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    bool ahead = false;  // lister: item i+1 was set up during the write-out of item i-1 already
    for (int i = 0;; ++i) {
      const int par = i & 1;
      if (ok) ok = mbar_wait_warp_idle(smem_u32(&sm->list_full[par]), (i >> 1) & 1, abort_flag, 256);
      const int w = ok ? *const_cast<volatile int*>(&sm->item[par]) : 0;
      if (w < 0) break;  // no more work: the same for all four warps
      const FwdItem it = fwd_item(w, p);
      const int n_tiles = ok ? *const_cast<volatile int*>(&sm->ntiles[par]) : 0;
      if (lister && ok && !ahead) {
        ok = mbar_wait_warp(smem_u32(&sm->setup_go[par]), (i >> 1) & 1, abort_flag);
        if (ok) set_up(i + 1);
      }
      ahead = false;
      if (ok) ok = mbar_wait_warp_idle(smem_u32(&sm->stats_full[par]), (i >> 1) & 1, abort_flag, 128);
      // The weights of the four partial results need the statistics only, which the softmax warps
      // publish before the item's last P V is complete: work them out before waiting for that, so
      // that the accumulators are given back (o_free) as soon as they have been read.
      float acc[64];
      float m_all = -INFINITY, l_all = 0.f, mt = -INFINITY, w0 = 0.f, w1 = 0.f;
      if (ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          m_all = fmaxf(m_all, sm->mref[par][j & 1][r_blk + 64 * (j >> 1)]);
          mt = fmaxf(mt, sm->mtrue[par][j & 1][r_blk + 64 * (j >> 1)]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float mi = sm->mref[par][j & 1][r_blk + 64 * (j >> 1)];
          if (mi != -INFINITY)
            l_all += ex2_approx(mi - m_all) * sm->lsum[par][j & 1][r_blk + 64 * (j >> 1)];
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        const float m0 = sm->mref[par][0][lane_row], m1 = sm->mref[par][1][lane_row];
        w0 = m0 == -INFINITY ? 0.f : ex2_approx(m0 - m_all) * inv;
        w1 = m1 == -INFINITY ? 0.f : ex2_approx(m1 - m_all) * inv;
      }
      if (ok) ok = mbar_wait_warp(smem_u32(&sm->o_full[par]), (i >> 1) & 1, abort_flag);
      if (ok) {
        if (n_tiles > 0) {  // warp-uniform
          // team 1's accumulator holds this item's sums only if the item has a tile c
          const bool live1 = n_tiles > 2;
          tc_fence_after();
#pragma unroll
          for (int part = 0; part < 4; ++part) {
            uint32_t a0[16], a1[16];
            tmem_ld_32x32b_x16(tmem + lane_base + kTmemO + 16 * part, a0);
            tmem_ld_32x32b_x16(tmem + lane_base + kTmemO + 64 + 16 * part, a1);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float x0 = __uint_as_float(a0[j]) * w0;
              acc[16 * part + j] = live1 ? fmaf(__uint_as_float(a1[j]), w1, x0) : x0;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j) acc[j] = 0.f;
        }
        // Accumulators, statistics and the item's header are in registers now: the next item may
        // use them, while this one is still being merged and stored.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->o_free[par]));
        // Lister: this item's list buffer is free now.  When the next item is already under way
        // and has asked for its successor (many items per CTA: it asks at once), set that one up
        // before merging and storing this item's rows: the write-out of an item ends late in the
        // next one, and a set-up that waited for it would itself be late for the one after.
        if (lister) {
          const int j = i + 1;
          if (__all_sync(0xffffffffu, mbar_test(smem_u32(&sm->setup_go[j & 1]), (j >> 1) & 1))) {
            set_up(j + 1);
            ahead = true;
          }
        }
      }
      const int row = it.mb * 64 + r_blk;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o) + it.b * p.o_sb +
                                            it.h * p.o_sh + static_cast<int64_t>(row) * p.o_sn);
      bool any_failed = false;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        if (ok && half == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) sm->xfer[j][r_blk] = acc[32 * part + j];
        }
        named_barrier_sync(2, 128);
        if (ok && half == 0) {
#pragma unroll
          for (int v8 = 0; v8 < 2; ++v8) {
            uint32_t pkd[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int col = 16 * v8 + 2 * j;
              pkd[j] = pack_2x16<kBf16>(acc[32 * part + col] + sm->xfer[col][r_blk],
                                        acc[32 * part + col + 1] + sm->xfer[col + 1][r_blk]);
            }
            // whole 32-byte sectors when the rows start on such boundaries
            if (p.wide_stores) {
              st_global_v8(dst + 4 * part + 2 * v8, pkd);
            } else {
              dst[4 * part + 2 * v8] = make_uint4(pkd[0], pkd[1], pkd[2], pkd[3]);
              dst[4 * part + 2 * v8 + 1] = make_uint4(pkd[4], pkd[5], pkd[6], pkd[7]);
            }
          }
        }
        // xfer may be overwritten now; all four warps leave together if any gave up
        any_failed = named_barrier_or(2, 128, !ok);
      }
      if (ok && half == 0) {
        const int64_t ri = (static_cast<int64_t>(it.b) * p.H + it.h) * p.N + row;
        p.lse2[ri] = l_all > 0.f ? m_all + lg2_approx(l_all) : -INFINITY;
        if (p.rowmax) p.rowmax[ri] = mt;
      }
      if (any_failed) break;
    }
    if (!ok) fwd_give_up(sm, p.status, kFailOut);
    if (lister && !terminal && lane == 0) {
      // gave up before the last draw: draw on (without working) until this CTA's first ticket past
      // the end, so that the launch still draws `items` tickets and the counter returns to zero
      int t;
      do {
        t = atomicAdd(p.ticket, 1);
        if (t == p.items - 1) atomicExch(p.ticket, 0);
      } while (t < n2);
    }

  }

  // ---- tear-down: every role arrives here, also after a give-up ----
  tc_fence_before();
  __syncthreads();
  if (warp == kSWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

// Tensor maps of recent operands.  Encoding one takes the driver about a microsecond, and a
// forward call needs three; a model calls the op with the same few buffers over and over.
struct TmapKey {
  const void* base;
  int64_t s[4];
  int B, H, N, dtype;
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};

static int cached_qkv_tmap(CUtensorMap* out, const void* base, const int64_t s[4], int B, int H,
                           int N, int dtype) {
  constexpr int kEntries = 12;
  static thread_local TmapEntry cache[kEntries];
  static thread_local int next = 0;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  for (int i = 0; i < 4; ++i) key.s[i] = s[i];
  key.B = B;
  key.H = H;
  key.N = N;
  key.dtype = dtype;
  for (int i = 0; i < kEntries; ++i)
    if (cache[i].valid && memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
      *out = cache[i].map;
      return BSA_OK;
    }
  const int rc = make_qkv_tmap(out, base, s, B, H, N, dtype, 64);
  if (rc != BSA_OK) return rc;
  TmapEntry& e = cache[next];
  next = (next + 1) % kEntries;
  e.key = key;
  e.map = *out;
  e.valid = true;
  return BSA_OK;
}

static int launch_fwd(const void* q, const int64_t q_strides[4], const void* k,
                      const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* o,
                      const int64_t o_strides[4], float* lse2, float* rowmax,
                      const int32_t* row_ptr, const int32_t* col_idx, const uint8_t* block,
                      const int64_t* block_strides, int list_b_stride, int list_h_stride,
                      float sm_scale, int dtype, int B, int H, int N, int D, int row_begin,
                      int row_end, const uint8_t* dense, const int64_t* dense_strides,
                      int32_t* status, int32_t* ticket, void* stream) {
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (!(sm_scale >= 0.f)) return BSA_ERR_BAD_SHAPE;  // the row maximum is taken before scaling
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!lse2 || (block == nullptr && (!row_ptr || !col_idx))) return BSA_ERR_BAD_POINTER;
  if (dense != nullptr) {
    // rows of 64 mask bytes are read as four 16-byte words; -inf times a zero scale would be NaN
    if (!dense_strides || !is_aligned(dense, 16)) return BSA_ERR_BAD_POINTER;
    if (dense_strides[3] != 1 || dense_strides[2] <= 0 || (dense_strides[2] % 16) != 0 ||
        dense_strides[0] < 0 || dense_strides[1] < 0 || (dense_strides[0] % 16) != 0 ||
        (dense_strides[1] % 16) != 0)
      return BSA_ERR_BAD_STRIDE;
    if (!(sm_scale > 0.f)) return BSA_ERR_BAD_SHAPE;
  }
  int rc;
  if ((rc = check_qkv_operand(q, q_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(k, k_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(v, v_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(o, o_strides)) != BSA_OK) return rc;
  if ((rc = check_device_sm100()) != BSA_OK) return rc;

  const int nb = N / kBlock;
  if (nb > kFwdMaxTiles) return BSA_ERR_TOO_LARGE;
  if (row_begin < 0 || row_end > nb || row_begin > row_end) return BSA_ERR_BAD_SHAPE;
  const int nrows = row_end - row_begin;
  if (nrows == 0) return BSA_OK;  // an empty share of the rows: nothing to launch
  if (static_cast<int64_t>(B) * H * nrows > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = cached_qkv_tmap(&tm_q, q, q_strides, B, H, N, dtype)) != BSA_OK) return rc;
  if ((rc = cached_qkv_tmap(&tm_k, k, k_strides, B, H, N, dtype)) != BSA_OK) return rc;
  if ((rc = cached_qkv_tmap(&tm_v, v, v_strides, B, H, N, dtype)) != BSA_OK) return rc;

  FwdParams prm;
  prm.row_ptr = row_ptr;
  prm.col_idx = col_idx;
  prm.block = block;
  prm.ms0 = block ? block_strides[0] : 0;
  prm.ms1 = block ? block_strides[1] : 0;
  prm.ms2 = block ? block_strides[2] : 0;
  prm.ms3 = block ? block_strides[3] : 0;
  prm.dense = dense;
  prm.ds0 = dense ? dense_strides[0] : 0;
  prm.ds1 = dense ? dense_strides[1] : 0;
  prm.ds2 = dense ? dense_strides[2] : 0;
  prm.o = o;
  prm.o_sb = o_strides[0];
  prm.o_sh = o_strides[1];
  prm.o_sn = o_strides[2];
  prm.lse2 = lse2;
  prm.rowmax = rowmax;
  prm.B = B;
  prm.H = H;
  prm.N = N;
  prm.nb = nb;
  prm.row_begin = row_begin;
  prm.nrows = nrows;
  prm.list_b_stride = list_b_stride;
  prm.list_h_stride = list_h_stride;
  prm.items = B * H * nrows;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.status = status;
  prm.ticket = ticket;
  prm.wide_stores =
      ((reinterpret_cast<uintptr_t>(o) |
        static_cast<uintptr_t>((o_strides[0] | o_strides[1] | o_strides[2]) * 2)) & 31u) == 0 ? 1 : 0;
  int sms = 0;
  if ((rc = sm_count(&sms)) != BSA_OK) return rc;

  const size_t smem_bytes = sizeof(FwdSmem) + 1024;
  auto kern = dense != nullptr
                  ? (dtype == BSA_BF16 ? attn_fwd_kernel<true, true> : attn_fwd_kernel<false, true>)
                  : (dtype == BSA_BF16 ? attn_fwd_kernel<true, false> : attn_fwd_kernel<false, false>);
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) != BSA_OK)
    return rc;
  const dim3 grid(static_cast<unsigned>(prm.items < sms ? prm.items : sms));  // one CTA per SM
  kern<<<grid, kFwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, prm);
  if (cudaGetLastError() != cudaSuccess) return BSA_ERR_CUDA;
  return BSA_OK;
}

}  // namespace bsa

extern "C" int bsa_attn_fwd_rows(const void* q, const int64_t q_strides[4], const void* k,
                                 const int64_t k_strides[4], const void* v,
                                 const int64_t v_strides[4], void* o, const int64_t o_strides[4],
                                 float* lse2, float* rowmax, const int32_t* row_ptr,
                                 const int32_t* col_idx, int list_b_stride, int list_h_stride,
                                 float sm_scale, int dtype, int B, int H, int N, int D,
                                 int row_begin, int row_end, const uint8_t* dense,
                                 const int64_t dense_strides[4], int32_t* work_counter,
                                 int32_t* status, void* stream) {
  if (!row_ptr || !col_idx) return BSA_ERR_BAD_POINTER;
  return bsa::launch_fwd(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, rowmax,
                         row_ptr, col_idx, nullptr, nullptr, list_b_stride, list_h_stride, sm_scale,
                         dtype, B, H, N, D, row_begin, row_end, dense, dense_strides, status,
                         work_counter, stream);
}

extern "C" int bsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k,
                            const int64_t k_strides[4], const void* v, const int64_t v_strides[4],
                            void* o, const int64_t o_strides[4], float* lse2, float* rowmax,
                            const int32_t* row_ptr, const int32_t* col_idx, int list_b_stride,
                            int list_h_stride, float sm_scale, int dtype, int B, int H, int N,
                            int D, int32_t* work_counter, int32_t* status, void* stream) {
  return bsa_attn_fwd_rows(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, rowmax,
                           row_ptr, col_idx, list_b_stride, list_h_stride, sm_scale, dtype, B, H,
                           N, D, 0, N / bsa::kBlock, nullptr, nullptr, work_counter, status, stream);
}

extern "C" int bsa_attn_fwd_block_mask_rows(
    const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
    const void* v, const int64_t v_strides[4], void* o, const int64_t o_strides[4], float* lse2,
    float* rowmax, const uint8_t* block, const int64_t block_strides[4], int Bm, int Hm,
    float sm_scale, int dtype, int B, int H, int N, int D, int row_begin, int row_end,
    const uint8_t* dense, const int64_t dense_strides[4], int32_t* work_counter, int32_t* status,
    void* stream) {
  if (!block || !block_strides) return BSA_ERR_BAD_POINTER;
  if ((Bm != 1 && Bm != B) || (Hm != 1 && Hm != H)) return BSA_ERR_BAD_SHAPE;
  for (int i = 0; i < 4; ++i)
    if (block_strides[i] < 0) return BSA_ERR_BAD_STRIDE;
  return bsa::launch_fwd(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, rowmax,
                         nullptr, nullptr, block, block_strides, Bm > 1 ? 1 : 0, Hm > 1 ? 1 : 0,
                         sm_scale, dtype, B, H, N, D, row_begin, row_end, dense, dense_strides,
                         status, work_counter, stream);
}

extern "C" int bsa_attn_fwd_block_mask(const void* q, const int64_t q_strides[4], const void* k,
                                       const int64_t k_strides[4], const void* v,
                                       const int64_t v_strides[4], void* o,
                                       const int64_t o_strides[4], float* lse2, float* rowmax,
                                       const uint8_t* block, const int64_t block_strides[4],
                                       int Bm, int Hm, float sm_scale, int dtype, int B, int H,
                                       int N, int D, int32_t* work_counter, int32_t* status,
                                       void* stream) {
  return bsa_attn_fwd_block_mask_rows(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2,
                                      rowmax, block, block_strides, Bm, Hm, sm_scale, dtype, B, H,
                                      N, D, 0, N > 0 ? N / bsa::kBlock : 0, nullptr, nullptr,
                                      work_counter, status, stream);
}
