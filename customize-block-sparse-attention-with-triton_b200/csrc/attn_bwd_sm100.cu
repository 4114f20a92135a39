// Backward block-sparse attention for sm_100a: one kernel template, two instantiations.
//
//   dK/dV (kDKDV = true):  a CTA owns ONE key block (64 keys), keeps its K and V in shared memory,
//       each loaded twice (rows 0..63 and 64..127 of the tcgen05 A operands), and walks the
//       block's list of query blocks (the column lists of the mask) two at a time ("supersteps"):
//         S^T = [K;K] [Q_a;Q_b]^T, dP^T = [V;V] [dO_a;dO_b]^T   (SS MMAs, M=128, N=128)
//       so that TMEM lanes 0..63 hold query tile a (columns 0..63) and lanes 64..127 query tile b
//       (columns 64..127): every SM sub-partition has exponentials to do whatever the mask is.
//         P^T = exp2(S^T c - LSE2[q]), dS^T = P^T (dP^T - delta[q])     (one thread per key row)
//         dV += P^T_a dO_a + P^T_b dO_b,  dK += dS^T_a Q_a + dS^T_b Q_b (TS MMAs: A from TMEM, B
//       MN-major from shared memory).  The half of the lanes that does not own a tile holds zeros
//       where that tile's P^T / dS^T live, so lane r sums the tile-a products of key r and lane
//       r+64 its tile-b products; the two are added when the block is written out.
//   dQ    (kDKDV = false): a CTA owns one query block, keeps Q and dO resident (twice) and walks the
//       row list of key blocks two at a time:
//         S = [Q;Q] [K_a;K_b]^T, dP = [dO;dO] [V_a;V_b]^T;  dS = exp2(S c - LSE2[row]) (dP - delta[row]);
//         dQ += dS_a K_a + dS_b K_b
//
// Formulas are those of the reference's backward (fa2_custom_mask/fa2_bwd.py:56-74, 116-130) with
// M replaced by a true base-2 log-sum-exp; the iteration space is the tile lists, not the
// reference's causal loops.  dK and dQ carry the factor sm_scale.
//
// Persistent: one CTA per SM starts with block blockIdx.x and draws further blocks from an
// optional work counter (or walks a fixed stride); long lists first when the mask is causal.
// Roles: warps 0..15 compute (lane quarter = warp % 4, 16 of a tile's 64 columns = warp / 4: four
// warps per SM sub-partition, so that one warp's TMEM loads, stores and barrier round trips hide
// behind the others' arithmetic), warp 16 TMA producer, warp 17 issues the S/dP MMAs and owns
// TMEM, warp 18 issues the accumulating MMAs (two issuers, so neither waits behind the other's
// barrier round trips; both run warp-wide with one elected lane issuing), warps 19..22 write a
// block's sums out while the compute warps are already at work on the next block.  S/dP are released as soon as the compute warps hold them in registers;
// P^T/dS^T live in their own TMEM buffers until the accumulating MMAs that read them are complete.
// Every wait is bounded and every barrier is waited on by warps that see each of its phases.
#include <math.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace bsa {

constexpr int kBwdStages = 4;
constexpr int kCW = 16;                    // compute warps: 4 lane quarters x (kCW / 4) column parts
constexpr int kChunk = 64 / (kCW / 4);     // columns of a tile per compute warp
constexpr int kProdWarp = kCW, kXWarp = kCW + 1, kAccWarp = kCW + 2;
constexpr int kBwdThreads = 32 * (kCW + 7);  // ... and four write-out warps (lane quarter = warp % 4)
constexpr uint32_t kBwdTile = 64 * 64 * 2;
constexpr uint32_t kBwdTmemCols = 512;
constexpr int kListIndex = BSA_LIST_PARTIAL_FLAG - 1;  // a list entry without its flag
// TMEM columns: X0 = S (or S^T), X1 = dP (or dP^T), 128 each (tile a in columns 0..63 of lanes
// 0..63, tile b in columns 64..127 of lanes 64..127); P and dS as 16-bit pairs, 32 columns per
// tile; two fp32 accumulators.
constexpr uint32_t kTmX0 = 0, kTmX1 = 128, kTmP = 256, kTmDS = 320, kTmAcc0 = 384, kTmAcc1 = 448;

struct BwdSmem {
  uint8_t stat0[2][kBwdTile];               // the CTA's own block, twice: K (dK/dV) or Q (dQ)
  uint8_t stat1[2][kBwdTile];               // V or dO, twice
  uint8_t str0[kBwdStages][2][kBwdTile];    // streamed tiles a, b: Q (dK/dV) or K (dQ)
  uint8_t str1[kBwdStages][2][kBwdTile];    // dO or V
  float lse[kBwdStages][2][64];             // dK/dV: LSE2 and delta of the streamed query tiles
  float delta[kBwdStages][2][64];
  // write-out hand-over, [col][row]: 0 = lanes 64..127 of the first (or only) accumulator, 1 =
  // lanes 64..127 of the second, 2 = lanes 0..63 of the second
  float xfer[3][64][65];
  int item[2];                              // by item parity: the work item, -1 = no more work
  int item_tiles[2], item_begin[2];         // ... its list length and where its list begins
  uint64_t item_full[2], item_free[2];      // header published; header read by all ten readers
  uint64_t stat_full, stat_free;            // own operands loaded; their S/dP instructions complete
  uint64_t acc_done;                        // all accumulating MMAs of the block complete
  uint64_t acc_free;                        // the write-out warps have read the accumulators
  uint64_t in_full[kBwdStages];
  uint64_t in_empty[kBwdStages];            // accumulating MMAs of the superstep complete
  uint64_t x_full, x_free;                  // S/dP complete; S/dP in the compute warps' registers
  uint64_t d_full, d_free;                  // P/dS stored; accumulating MMAs that read them complete
  uint32_t tmem_base;
  int abort_flag;
};

static_assert(sizeof(BwdSmem) + 1024 <= 232448, "BwdSmem exceeds the shared memory of one CTA");

struct BwdParams {
  const int32_t* list_ptr;  // dK/dV: column lists (col_ptr/row_idx); dQ: row lists (row_ptr/col_idx)
  const int32_t* list_idx;
  const uint8_t* dense;     // optional element-level mask for the tiles whose list entry is flagged
  int64_t ds0, ds1, ds2;
  const float* lse2;
  const float* delta;
  void* out0;  // dV (dK/dV kernel only)
  void* out1;  // dK or dQ
  int64_t sb, sh, sn;
  int B, H, N, nb;
  int items;  // B * H * nb
  int list_b_stride, list_h_stride;
  float scale_log2;
  float sm_scale;
  int32_t* status;
  int32_t* ticket;  // optional work counter (0 at kernel start, left 0): dynamic item hand-out
  int wide_stores;  // output rows start on 32-byte boundaries
};

__device__ __forceinline__ void bwd_give_up(BwdSmem* sm, int32_t* status, int code) {
  sm->abort_flag = 1;
  report_status(status, code);
}

// Stores 32 columns of one output row: (own[c] + other[c]) * scale as 16-bit; `other` walks the
// hand-over buffer ([col][row], 65 floats per column).
// (wide: the rows start on 32-byte boundaries, so 16 columns go out as one whole sector)
template <bool kBf16>
__device__ __forceinline__ void store_cols32(void* base, int64_t elem_off, const uint32_t* own,
                                             const float* other, float scale, bool wide) {
  uint16_t* dst = static_cast<uint16_t*>(base) + elem_off;
#pragma unroll
  for (int v = 0; v < 2; ++v) {
    uint32_t w[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int c = 16 * v + 2 * t;
      w[t] = pack_2x16<kBf16>((__uint_as_float(own[c]) + other[c * 65]) * scale,
                              (__uint_as_float(own[c + 1]) + other[(c + 1) * 65]) * scale);
    }
    if (wide) {
      st_global_v8(dst + 16 * v, w);
    } else {
      reinterpret_cast<uint4*>(dst + 16 * v)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(dst + 16 * v)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

// Readers of the item header: wait for item i, read it (the producer looked the list up, so the
// other roles start an item without a round trip to memory), tell the producer the slot was read.
__device__ __forceinline__ bool bwd_next_item(BwdSmem* sm, int i, int lane, volatile int* abort_flag,
                                              int* w, int* n_tiles, int* begin) {
  const int par = i & 1;
  if (!mbar_wait_warp(smem_u32(&sm->item_full[par]), (i >> 1) & 1, abort_flag)) return false;
  *w = *const_cast<volatile int*>(&sm->item[par]);
  *n_tiles = *const_cast<volatile int*>(&sm->item_tiles[par]);
  *begin = *const_cast<volatile int*>(&sm->item_begin[par]);
  __syncwarp();
  if (lane == 0) mbar_arrive(smem_u32(&sm->item_free[par]));
  return true;
}

// Work item w -> (batch, head, block) and the block's list.
// dQ: long (late) rows first; dK/dV: long (early) key columns first when the mask is causal.
struct BwdItem {
  int b, h, blk, n_tiles;
  const int32_t* ents;
  int64_t vec_base;  // into lse2 / delta
};
// (n_tiles < 0: look the list up; otherwise the caller has its length and beginning already)
template <bool kDKDV>
__device__ __forceinline__ BwdItem bwd_item(int w, const BwdParams& p, int n_tiles = -1,
                                            int begin = 0) {
  BwdItem it;
  const int bh = w / p.nb;
  it.blk = kDKDV ? (w - bh * p.nb) : (p.nb - 1 - (w - bh * p.nb));
  it.b = bh / p.H;
  it.h = bh - it.b * p.H;
  if (n_tiles < 0) {
    const int64_t li =
        static_cast<int64_t>(it.b * p.list_b_stride + it.h * p.list_h_stride) * p.nb + it.blk;
    begin = __ldg(p.list_ptr + li);
    n_tiles = __ldg(p.list_ptr + li + 1) - begin;
  }
  it.n_tiles = n_tiles;
  it.ents = p.list_idx + begin;
  it.vec_base = (static_cast<int64_t>(it.b) * p.H + it.h) * p.N;
  return it;
}

// Persistent: one CTA per SM.  The producer starts with item blockIdx.x and then draws further
// items from the optional work counter (or walks a fixed stride), and hands each item's index to
// the other roles through shared memory; every role walks the same sequence and counts
// supersteps (gs) and non-empty items (ni) the same way, so barrier phases follow from the counts.

// kElementMask: the instantiation that applies a dense mask inside the tiles whose list entries
// are flagged; the plain one carries none of that code.
template <bool kBf16, bool kDKDV, bool kElementMask>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_stat0,
                const __grid_constant__ CUtensorMap tm_stat1,
                const __grid_constant__ CUtensorMap tm_str0,
                const __grid_constant__ CUtensorMap tm_str1, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  BwdSmem* sm = reinterpret_cast<BwdSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;
  const int stride = gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm->item_full[i]), 1);
      mbar_init(smem_u32(&sm->item_free[i]), kCW + 6);  // compute warps, two issuers, four write-out warps
    }
    mbar_init(smem_u32(&sm->stat_full), 1);
    mbar_init(smem_u32(&sm->stat_free), 1);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(smem_u32(&sm->in_full[s]), 1);
      mbar_init(smem_u32(&sm->in_empty[s]), 1);
    }
    mbar_init(smem_u32(&sm->x_full), 1);
    mbar_init(smem_u32(&sm->x_free), kCW);  // one arrival per compute warp
    mbar_init(smem_u32(&sm->d_full), kCW);
    mbar_init(smem_u32(&sm->d_free), 1);
    mbar_init(smem_u32(&sm->acc_done), 1);
    mbar_init(smem_u32(&sm->acc_free), 4);  // one arrival per write-out warp
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kXWarp) {
    tmem_alloc(smem_u32(&sm->tmem_base), kBwdTmemCols);
    tmem_relinquish();
  }
  if (warp == kProdWarp && lane == 0) {
    tma_prefetch_desc(&tm_stat0);
    tma_prefetch_desc(&tm_stat1);
    tma_prefetch_desc(&tm_str0);
    tma_prefetch_desc(&tm_str1);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->abort_flag;

  if (warp == kProdWarp) {
    // =========================== TMA producer ===========================
    bool ok = true;
    bool terminal = p.ticket == nullptr;  // drew a ticket past the end (or draws none)
    int gs = 0, ni = 0;
    for (int i = 0, w = blockIdx.x; ok; ++i) {
      const int par = i & 1;
      if (i > 0) {
        if (p.ticket != nullptr) {
          int t = 0;
          if (lane == 0) {
            t = atomicAdd(p.ticket, 1);
            // every CTA draws until its first ticket past the end, so the launch draws exactly
            // `items` tickets in all; whoever draws the last one leaves the counter at zero
            if (t == p.items - 1) atomicExch(p.ticket, 0);
          }
          w = stride + __shfl_sync(0xffffffffu, t, 0);
          terminal = w >= p.items;
        } else {
          w += stride;
        }
      }
      // the header slot of item i-2 must have been read by everyone
      if (i >= 2)
        ok = mbar_wait_warp(smem_u32(&sm->item_free[par]), ((i - 2) >> 1) & 1, abort_flag);
      if (!ok) break;
      BwdItem it;
      it.n_tiles = 0;
      if (w < p.items) it = bwd_item<kDKDV>(w, p);
      if (lane == 0) {
        sm->item[par] = w < p.items ? w : -1;
        sm->item_tiles[par] = it.n_tiles;
        sm->item_begin[par] = w < p.items ? static_cast<int>(it.ents - p.list_idx) : 0;
        mbar_arrive(smem_u32(&sm->item_full[par]));  // release: the header is visible
      }
      if (w >= p.items) break;
      const int n_super = (it.n_tiles + 1) >> 1;
      if (n_super == 0) continue;
      // the block's own operands: the previous item's S/dP instructions must be complete
      if (ni >= 1) ok = mbar_wait_warp(smem_u32(&sm->stat_free), (ni - 1) & 1, abort_flag);
      if (!ok) break;
      // One lane per copy: a single thread can start a tile load only every couple of hundred
      // cycles, which up to eight copies in a row would turn into the kernel's bound.
      {
        const uint32_t bar = smem_u32(&sm->stat_full);
        if (lane == 0) mbar_expect_tx(bar, 4 * kBwdTile);
        __syncwarp();
        if (lane < 2)
          tma_load_4d(smem_u32(sm->stat0[lane]), &tm_stat0, bar, 0, it.blk * 64, it.h, it.b);
        else if (lane < 4)
          tma_load_4d(smem_u32(sm->stat1[lane - 2]), &tm_stat1, bar, 0, it.blk * 64, it.h, it.b);
      }
      for (int j = 0; j < n_super; ++j, ++gs) {
        const int s = gs % kBwdStages;
        const int nt = min(2, it.n_tiles - 2 * j);
        const int tl = (lane >> 1) & 1;  // lanes 0, 1, 4, 5 serve tile a, lanes 2, 3, 6, 7 tile b
        const int nj = tl < nt ? (__ldg(it.ents + 2 * j + tl) & kListIndex) : 0;
        ok = mbar_wait_warp(smem_u32(&sm->in_empty[s]), ((gs / kBwdStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        const uint32_t bar = smem_u32(&sm->in_full[s]);
        if (lane == 0) mbar_expect_tx(bar, nt * (2 * kBwdTile + (kDKDV ? 512u : 0u)));
        __syncwarp();
        if (tl < nt) {
          if (lane < 4) {
            if (lane & 1)
              tma_load_4d(smem_u32(sm->str1[s][tl]), &tm_str1, bar, 0, nj * 64, it.h, it.b);
            else
              tma_load_4d(smem_u32(sm->str0[s][tl]), &tm_str0, bar, 0, nj * 64, it.h, it.b);
          } else if (kDKDV && lane < 8) {
            if (lane & 1)
              bulk_load_1d(smem_u32(sm->delta[s][tl]), p.delta + it.vec_base + nj * 64, 256, bar);
            else
              bulk_load_1d(smem_u32(sm->lse[s][tl]), p.lse2 + it.vec_base + nj * 64, 256, bar);
          }
        }
      }
      ++ni;
    }
    if (!ok) bwd_give_up(sm, p.status, 1);
    if (!terminal && lane == 0) {
      // gave up before the last draw: draw on (without working) until this CTA's first ticket past
      // the end, so that the launch still draws `items` tickets and the counter returns to zero
      int t;
      do {
        t = atomicAdd(p.ticket, 1);
        if (t == p.items - 1) atomicExch(p.ticket, 0);
      } while (stride + t < p.items);
    }
  } else if (warp == kXWarp) {
    // =========================== S / dP issuer ===========================
    constexpr uint32_t idesc_x128 = umma_idesc(kBf16, 0, 0, 128, 128);
    constexpr uint32_t idesc_x64 = umma_idesc(kBf16, 0, 0, 128, 64);  // odd tail: one tile
    const bool leader = elect_one();
    const uint64_t desc_a0 = smem_desc_sw128(smem_u32(sm->stat0[0]), 16, 1024);
    const uint64_t desc_a1 = smem_desc_sw128(smem_u32(sm->stat1[0]), 16, 1024);
    const uint64_t desc_b0 = smem_desc_sw128(smem_u32(sm->str0[0][0]), 16, 1024);
    const uint64_t desc_b1 = smem_desc_sw128(smem_u32(sm->str1[0][0]), 16, 1024);
    bool ok = true;
    int gs = 0, ni = 0;
    for (int i = 0; ok; ++i) {
      int w, w_tiles, w_begin;
      ok = bwd_next_item(sm, i, lane, abort_flag, &w, &w_tiles, &w_begin);
      if (!ok || w < 0) break;
      const BwdItem it = bwd_item<kDKDV>(w, p, w_tiles, w_begin);
      const int n_super = (it.n_tiles + 1) >> 1;
      if (n_super == 0) continue;
      ok = mbar_wait_warp(smem_u32(&sm->stat_full), ni & 1, abort_flag);
      for (int j = 0; ok && j < n_super; ++j, ++gs) {
        const int s = gs % kBwdStages;
        const int nt = min(2, it.n_tiles - 2 * j);
        ok = mbar_wait_warp(smem_u32(&sm->in_full[s]), (gs / kBwdStages) & 1, abort_flag);
        if (!ok) break;
        // S/dP of the previous superstep must be in the compute warps' registers (for the first
        // one this asks for the phase before the first one, which counts as complete)
        ok = mbar_wait_warp(smem_u32(&sm->x_free), (gs & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          const uint64_t b0 = desc_b0 + static_cast<uint64_t>(s * ((2 * kBwdTile) >> 4));
          const uint64_t b1 = desc_b1 + static_cast<uint64_t>(s * ((2 * kBwdTile) >> 4));
          const uint32_t idesc = nt == 2 ? idesc_x128 : idesc_x64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + kTmX0, desc_a0 + 2 * kk, b0 + 2 * kk, idesc, kk > 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + kTmX1, desc_a1 + 2 * kk, b1 + 2 * kk, idesc, kk > 0);
          tc_commit(smem_u32(&sm->x_full));
          if (j == n_super - 1) tc_commit(smem_u32(&sm->stat_free));  // own operands reusable
        }
      }
      ++ni;
    }
    if (!ok) bwd_give_up(sm, p.status, 2);
  } else if (warp == kAccWarp) {
    // =========================== accumulating-MMA issuer ===========================
    constexpr uint32_t idesc_acc = umma_idesc(kBf16, 0, 1, 128, 64);
    const bool leader = elect_one();
    const uint64_t desc_m0 = smem_desc_sw128(smem_u32(sm->str0[0][0]), 8192, 1024);
    const uint64_t desc_m1 = smem_desc_sw128(smem_u32(sm->str1[0][0]), 8192, 1024);
    bool ok = true;
    int gs = 0, ni = 0;
    for (int i = 0; ok; ++i) {
      int w, w_tiles, w_begin;
      ok = bwd_next_item(sm, i, lane, abort_flag, &w, &w_tiles, &w_begin);
      if (!ok || w < 0) break;
      const BwdItem it = bwd_item<kDKDV>(w, p, w_tiles, w_begin);
      const int n_super = (it.n_tiles + 1) >> 1;
      if (n_super == 0) continue;
      // the write-out warps must have read the previous block's accumulators
      if (ni >= 1) ok = mbar_wait_warp(smem_u32(&sm->acc_free), (ni - 1) & 1, abort_flag);
      for (int j = 0; ok && j < n_super; ++j, ++gs) {
        const int s = gs % kBwdStages;
        const int nt = min(2, it.n_tiles - 2 * j);
        ok = mbar_wait_warp(smem_u32(&sm->d_full), gs & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          // keys/queries [16 kk, +16) of tile t sit at column 32 t + 8 kk of the P / dS buffers
          for (int t = 0; t < nt; ++t) {
            const uint32_t first = (j > 0 || t > 0) ? 1u : 0u;
            if constexpr (kDKDV) {
              const uint64_t bmn = desc_m1 + static_cast<uint64_t>((2 * s + t) * (kBwdTile >> 4));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_ts(tmem + kTmAcc0, tmem + kTmP + 32 * t + 8 * kk, bmn + 128 * kk, idesc_acc,
                        first | (kk > 0));
            }
            const uint64_t bmn = desc_m0 + static_cast<uint64_t>((2 * s + t) * (kBwdTile >> 4));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ts(tmem + kTmAcc1, tmem + kTmDS + 32 * t + 8 * kk, bmn + 128 * kk, idesc_acc,
                      first | (kk > 0));
          }
          tc_commit(smem_u32(&sm->in_empty[s]));  // stage free
          tc_commit(smem_u32(&sm->d_free));       // P/dS buffers free; accumulators updated
          if (j == n_super - 1) tc_commit(smem_u32(&sm->acc_done));  // the block's sums are final
        }
      }
      ++ni;
    }
    if (!ok) bwd_give_up(sm, p.status, 2);
  } else if (warp < kCW) {
    // =========================== compute warps ===========================
    const int quarter = warp & 3;
    const int ch = warp >> 2;           // which kChunk of the tile's 64 columns
    const int t_mine = quarter >> 1;    // lanes 0..63 own tile a of a superstep, 64..127 tile b
    const int r_blk = (quarter & 1) * 32 + lane;  // row of the CTA's block
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale_log2;
    {
      // The accumulating MMAs of a tile sweep all 128 lanes: the half of the lanes that does not
      // own the tile holds zeros where that tile's P / dS live.  Nothing else ever writes there.
      uint32_t z[kChunk / 2];
#pragma unroll
      for (int i = 0; i < kChunk / 2; ++i) z[i] = 0u;
      if constexpr (kDKDV)
        tmem_st_cols<kChunk / 2>(tmem + lane_base + kTmP + 32 * (1 - t_mine) + (kChunk / 2) * ch, z);
      tmem_st_cols<kChunk / 2>(tmem + lane_base + kTmDS + 32 * (1 - t_mine) + (kChunk / 2) * ch, z);
      tc_wait_st();
    }
    bool ok = true;
    int gs = 0;
    for (int i = 0; ok; ++i) {
      int w, w_tiles, w_begin;
      ok = bwd_next_item(sm, i, lane, abort_flag, &w, &w_tiles, &w_begin);
      if (!ok || w < 0) break;
      const BwdItem it = bwd_item<kDKDV>(w, p, w_tiles, w_begin);
      const int n_super = (it.n_tiles + 1) >> 1;
      const int row = it.blk * 64 + r_blk;
      if (n_super == 0) continue;  // (the write-out warps store the zero gradients)
      float my_lse = 0.f, my_delta = 0.f;
      if constexpr (!kDKDV) {
        // (a row whose elements are all masked has LSE = -inf; every logit it meets is -inf too,
        // and against a finite stand-in it exponentiates to 0 instead of NaN)
        my_lse = __ldg(p.lse2 + it.vec_base + row);
        if constexpr (kElementMask) my_lse = fmaxf(my_lse, -3.0e38f);
        my_delta = __ldg(p.delta + it.vec_base + row);
      }
      // element-level mask: where this lane's mask bytes of a tile start (dQ: its query row, 32
      // consecutive keys; dK/dV: its key column, 32 consecutive query rows)
      const uint8_t* mask_at = nullptr;
      if constexpr (kElementMask)
        mask_at = p.dense + it.b * p.ds0 + it.h * p.ds1 +
                  (kDKDV ? static_cast<int64_t>(row) : static_cast<int64_t>(row) * p.ds2);
      for (int j = 0; ok && j < n_super; ++j, ++gs) {
        const int s = gs % kBwdStages;
        const int nt = min(2, it.n_tiles - 2 * j);
        const bool active = t_mine < nt;  // warp-uniform
        // A tile with masked elements inside: fetch this lane's 32 mask bytes while S is on its way
        uint32_t mw[kChunk / 4];
        bool partial = false;
        if (kElementMask && active) {
          const int e = __ldg(it.ents + 2 * j + t_mine);
          partial = (e & BSA_LIST_PARTIAL_FLAG) != 0;  // warp-uniform
          if (partial) {
            const int64_t other = static_cast<int64_t>((e & kListIndex) * 64 + kChunk * ch);
            if constexpr (kDKDV) {
              const uint8_t* mp = mask_at + other * p.ds2;
#pragma unroll
              for (int q4 = 0; q4 < kChunk / 4; ++q4) {
                uint32_t w4 = 0;
#pragma unroll
                for (int bb = 0; bb < 4; ++bb)
                  w4 |= static_cast<uint32_t>(__ldg(mp + (4 * q4 + bb) * p.ds2)) << (8 * bb);
                mw[q4] = w4;
              }
            } else {
              const uint4* mp = reinterpret_cast<const uint4*>(mask_at + other);
#pragma unroll
              for (int q16 = 0; q16 < kChunk / 16; ++q16) {
                const uint4 a = __ldg(mp + q16);
                mw[4 * q16] = a.x; mw[4 * q16 + 1] = a.y; mw[4 * q16 + 2] = a.z; mw[4 * q16 + 3] = a.w;
              }
            }
          }
        }
        if constexpr (kDKDV) {
          // the LSE2/delta vectors of this stage arrive through the async proxy
          ok = mbar_wait_warp(smem_u32(&sm->in_full[s]), (gs / kBwdStages) & 1, abort_flag);
          if (!ok) break;
        }
        ok = mbar_wait_warp(smem_u32(&sm->x_full), gs & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        uint32_t xs[kChunk], xd[kChunk];
        if (active) {
          tmem_ld_cols<kChunk>(tmem + lane_base + kTmX0 + 64 * t_mine + kChunk * ch, xs);
          tmem_ld_cols<kChunk>(tmem + lane_base + kTmX1 + 64 * t_mine + kChunk * ch, xd);
        }
        tc_wait_ld();
        // S/dP are in registers: the next superstep's may be issued
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->x_free));
        if (partial) {
          // masked elements: logit -inf, so P = 0 and with it dS = 0
#pragma unroll
          for (int q4 = 0; q4 < kChunk / 4; ++q4) {
            const uint32_t nz = __vcmpne4(mw[q4], 0u);
#pragma unroll
            for (int bb = 0; bb < 4; ++bb) {
              const uint32_t keep = __byte_perm(nz, 0u, 0x1111u * bb);
              xs[4 * q4 + bb] = (xs[4 * q4 + bb] & keep) | (0xff800000u & ~keep);
            }
          }
        }
        uint32_t pk_p[kChunk / 2], pk_ds[kChunk / 2];
        if (active) {
          const float4* lse4 = reinterpret_cast<const float4*>(&sm->lse[s][t_mine][kChunk * ch]);
          const float4* del4 = reinterpret_cast<const float4*>(&sm->delta[s][t_mine][kChunk * ch]);
#pragma unroll
          for (int i = 0; i < kChunk; i += 4) {
            float l[4], d[4];
            if constexpr (kDKDV) {
              const float4 lv = lse4[i / 4], dv = del4[i / 4];
              // (-inf = a query row with every element masked: see my_lse above)
              l[0] = lv.x; l[1] = lv.y; l[2] = lv.z; l[3] = lv.w;
              if constexpr (kElementMask) {
#pragma unroll
                for (int t = 0; t < 4; ++t) l[t] = fmaxf(l[t], -3.0e38f);
              }
              d[0] = dv.x; d[1] = dv.y; d[2] = dv.z; d[3] = dv.w;
            } else {
              l[0] = l[1] = l[2] = l[3] = my_lse;
              d[0] = d[1] = d[2] = d[3] = my_delta;
            }
            // two columns per instruction where the operands allow it (same rounding as scalar)
            float pv[4], dsv[4];
#pragma unroll
            for (int t = 0; t < 4; t += 2) {
              const uint64_t dp2 =
                  pack_f32x2(__uint_as_float(xd[i + t]), __uint_as_float(xd[i + t + 1]));
              uint64_t diff2;
              if constexpr (kDKDV) {
                // LSE and delta differ from column to column here
                pv[t] = ex2_approx(fmaf(__uint_as_float(xs[i + t]), c, -l[t]));
                pv[t + 1] = ex2_approx(fmaf(__uint_as_float(xs[i + t + 1]), c, -l[t + 1]));
                diff2 = fma_f32x2(pack_f32x2(d[t], d[t + 1]), pack_f32x2(-1.f, -1.f), dp2);
              } else {
                float z0, z1;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(xs[i + t]),
                                                  __uint_as_float(xs[i + t + 1])),
                                       pack_f32x2(c, c), pack_f32x2(-my_lse, -my_lse)),
                             z0, z1);
                pv[t] = ex2_approx(z0);
                pv[t + 1] = ex2_approx(z1);
                diff2 = add_f32x2(dp2, pack_f32x2(-my_delta, -my_delta));
              }
              unpack_f32x2(mul_f32x2(pack_f32x2(pv[t], pv[t + 1]), diff2), dsv[t], dsv[t + 1]);
            }
            pk_p[i / 2] = pack_2x16<kBf16>(pv[0], pv[1]);
            pk_p[i / 2 + 1] = pack_2x16<kBf16>(pv[2], pv[3]);
            pk_ds[i / 2] = pack_2x16<kBf16>(dsv[0], dsv[1]);
            pk_ds[i / 2 + 1] = pack_2x16<kBf16>(dsv[2], dsv[3]);
          }
        }
        // the accumulating MMAs of the previous superstep still read the P/dS buffers
        ok = mbar_wait_warp(smem_u32(&sm->d_free), (gs & 1) ^ 1, abort_flag);
        if (!ok) break;
        if (active) {
          tc_fence_after();
          if constexpr (kDKDV)
            tmem_st_cols<kChunk / 2>(tmem + lane_base + kTmP + 32 * t_mine + (kChunk / 2) * ch, pk_p);
          tmem_st_cols<kChunk / 2>(tmem + lane_base + kTmDS + 32 * t_mine + (kChunk / 2) * ch, pk_ds);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm->d_full));
      }
      // (the block's sums are merged and stored by the write-out warps; these warps go straight
      // on to the next block, whose first S/dP is usually complete already)
    }
    if (!ok) bwd_give_up(sm, p.status, 3);
  } else {
    // =========================== write-out ===========================
    // Lane r of an accumulator holds the tile-a sums of row r of the CTA's block, lane r+64 its
    // tile-b sums (never unwritten, even for a single-tile list: the first accumulate-off MMA
    // sweeps all lanes, and theirs hold zeros for tile a).  These four warps (lane quarter = warp
    // % 4) take the sums out of tensor memory as soon as the block's last MMAs are complete, so
    // that the next block can start accumulating, then add the two halves, scale, round and
    // store, while the compute warps are already at work on the next block.  Lanes 64..127 pass
    // everything on through shared memory; for dK/dV lanes 0..63 pass their second accumulator
    // on as well, and the warps of lanes 64..127 merge and store that one.
    // Both named barriers of an iteration are always executed, also after a give-up, and the
    // last one carries the give-up vote, so that no warp of this role is left waiting at one.
    const int quarter = warp & 3;
    const int half = quarter >> 1;
    const int r_blk = (quarter & 1) * 32 + lane;  // row of the CTA's block
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tm_first = tmem + lane_base + (kDKDV ? kTmAcc0 : kTmAcc1);
    const uint32_t tm_second = tmem + lane_base + kTmAcc1;  // dK (dK/dV kernel only)
    void* const out_first = kDKDV ? p.out0 : p.out1;
    const float scale_first = kDKDV ? 1.0f : p.sm_scale;
    const bool wide = p.wide_stores != 0;
    bool ok = true;
    int ni = 0;
    for (int i = 0;; ++i) {
      int w = 0, w_tiles = 1, w_begin = 0;
      if (ok) ok = bwd_next_item(sm, i, lane, abort_flag, &w, &w_tiles, &w_begin);
      if (ok && w < 0) break;  // no more work: the same for all four warps
      const BwdItem it = bwd_item<kDKDV>(ok ? w : 0, p, ok ? w_tiles : 1, 0);
      const int n_super = (it.n_tiles + 1) >> 1;
      const int64_t off =
          it.b * p.sb + it.h * p.sh + static_cast<int64_t>(it.blk * 64 + r_blk) * p.sn;
      if (n_super == 0) {
        // a block with an empty list: zero gradients (the same decision in all four warps)
        if (half == 0 || kDKDV) {
          uint4* dst = reinterpret_cast<uint4*>(
              static_cast<uint16_t*>(half == 0 ? out_first : p.out1) + off);
#pragma unroll
          for (int v = 0; v < 8; ++v) dst[v] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      if (ok) ok = mbar_wait_warp(smem_u32(&sm->acc_done), ni & 1, abort_flag);
      ++ni;
      uint32_t own[32];
      if (ok) {
        tc_fence_after();
        if (half == 1) {
#pragma unroll
          for (int a = 0; a < (kDKDV ? 2 : 1); ++a) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              tmem_ld_32x32b_x32((a == 0 ? tm_first : tm_second) + 32 * h2, own);
              tc_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) sm->xfer[a][32 * h2 + c][r_blk] = __uint_as_float(own[c]);
            }
          }
        } else {
          if constexpr (kDKDV) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              tmem_ld_32x32b_x32(tm_second + 32 * h2, own);
              tc_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) sm->xfer[2][32 * h2 + c][r_blk] = __uint_as_float(own[c]);
            }
          }
          tmem_ld_32x32b_x32(tm_first, own);
          tc_wait_ld();
        }
        if (half == 1) {
          // everything of these lanes is out of tensor memory
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm->acc_free));
        }
      }
      named_barrier_sync(2, 128);
      if (ok) {
        if (half == 0) {
          store_cols32<kBf16>(out_first, off, own, &sm->xfer[0][0][r_blk], scale_first, wide);
          tmem_ld_32x32b_x32(tm_first + 32, own);
          tc_wait_ld();
          // the accumulators are out of tensor memory: the next block may start accumulating
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm->acc_free));
          store_cols32<kBf16>(out_first, off + 32, own, &sm->xfer[0][32][r_blk], scale_first, wide);
        } else if constexpr (kDKDV) {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
#pragma unroll
            for (int c = 0; c < 32; ++c) own[c] = __float_as_uint(sm->xfer[2][32 * h2 + c][r_blk]);
            store_cols32<kBf16>(p.out1, off + 32 * h2, own, &sm->xfer[1][32 * h2][r_blk],
                                p.sm_scale, wide);
          }
        }
      }
      // xfer may be overwritten by the next block now; all four warps leave together on a give-up
      if (named_barrier_or(2, 128, !ok)) break;
    }
    if (!ok) bwd_give_up(sm, p.status, 3);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kXWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

template <bool kDKDV>
static int launch_bwd(const void* q, const void* k, const void* v, const void* dout,
                      const int64_t strides[4], const float* lse2, const float* delta, void* out0,
                      void* out1, const int32_t* list_ptr, const int32_t* list_idx,
                      int list_b_stride, int list_h_stride, float sm_scale, int dtype, int B, int H,
                      int N, int D, const uint8_t* dense, const int64_t* dense_strides,
                      int32_t* ticket, int32_t* status, void* stream) {
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (dense != nullptr) {
    if (!dense_strides || !is_aligned(dense, 16)) return BSA_ERR_BAD_POINTER;
    if (dense_strides[3] != 1 || dense_strides[2] <= 0 || (dense_strides[2] % 16) != 0 ||
        dense_strides[0] < 0 || dense_strides[1] < 0 || (dense_strides[0] % 16) != 0 ||
        (dense_strides[1] % 16) != 0)
      return BSA_ERR_BAD_STRIDE;
    if (!(sm_scale > 0.f)) return BSA_ERR_BAD_SHAPE;
  }
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!lse2 || !delta || !list_ptr || !list_idx || !is_aligned(lse2, 16) || !is_aligned(delta, 16))
    return BSA_ERR_BAD_POINTER;
  int rc;
  const void* ops[6] = {q, k, v, dout, out1, kDKDV ? out0 : out1};
  for (const void* op : ops)
    if ((rc = check_qkv_operand(op, strides)) != BSA_OK) return rc;
  if ((rc = check_device_sm100()) != BSA_OK) return rc;
  const int nb = N / kBlock;
  if (static_cast<int64_t>(B) * H * nb > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  // dK/dV: K, V resident; Q, dO streamed.   dQ: Q, dO resident; K, V streamed.
  const void* stat0 = kDKDV ? k : q;
  const void* stat1 = kDKDV ? v : dout;
  const void* str0 = kDKDV ? q : k;
  const void* str1 = kDKDV ? dout : v;
  CUtensorMap tm_a0, tm_a1, tm_b0, tm_b1;
  if ((rc = make_qkv_tmap(&tm_a0, stat0, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_a1, stat1, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_b0, str0, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_b1, str1, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;

  BwdParams prm;
  prm.list_ptr = list_ptr;
  prm.list_idx = list_idx;
  prm.dense = dense;
  prm.ds0 = dense ? dense_strides[0] : 0;
  prm.ds1 = dense ? dense_strides[1] : 0;
  prm.ds2 = dense ? dense_strides[2] : 0;
  prm.lse2 = lse2;
  prm.delta = delta;
  prm.out0 = out0;
  prm.out1 = out1;
  prm.sb = strides[0];
  prm.sh = strides[1];
  prm.sn = strides[2];
  prm.B = B;
  prm.H = H;
  prm.N = N;
  prm.nb = nb;
  prm.items = B * H * nb;
  prm.list_b_stride = list_b_stride;
  prm.list_h_stride = list_h_stride;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.sm_scale = sm_scale;
  prm.status = status;
  prm.ticket = ticket;
  {
    // a thread's 16 output columns are one 32-byte sector when every row starts on such a boundary
    const uintptr_t bits = reinterpret_cast<uintptr_t>(out0) | reinterpret_cast<uintptr_t>(out1);
    const int64_t sbits = (strides[0] | strides[1] | strides[2]) * 2;
    prm.wide_stores = ((bits | static_cast<uintptr_t>(sbits)) & 31u) == 0 ? 1 : 0;
  }

  const size_t smem_bytes = sizeof(BwdSmem) + 1024;
  auto kern = dense != nullptr ? (dtype == BSA_BF16 ? attn_bwd_kernel<true, kDKDV, true>
                                                    : attn_bwd_kernel<false, kDKDV, true>)
                               : (dtype == BSA_BF16 ? attn_bwd_kernel<true, kDKDV, false>
                                                    : attn_bwd_kernel<false, kDKDV, false>);
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) != BSA_OK)
    return rc;
  int sms = 0;
  if ((rc = sm_count(&sms)) != BSA_OK) return rc;
  const dim3 grid(static_cast<unsigned>(prm.items < sms ? prm.items : sms));  // one CTA per SM
  kern<<<grid, kBwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm_a0, tm_a1, tm_b0,
                                                                             tm_b1, prm);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}

}  // namespace bsa

extern "C" int bsa_attn_bwd_dkdv(const void* q, const void* k, const void* v, const void* dout,
                                 const int64_t strides[4], const float* lse2, const float* delta,
                                 void* dk, void* dv, const int32_t* col_ptr,
                                 const int32_t* row_idx, int list_b_stride, int list_h_stride,
                                 float sm_scale, int dtype, int B, int H, int N, int D,
                                 const uint8_t* dense, const int64_t dense_strides[4],
                                 int32_t* work_counter, int32_t* status, void* stream) {
  return bsa::launch_bwd<true>(q, k, v, dout, strides, lse2, delta, dv, dk, col_ptr, row_idx,
                               list_b_stride, list_h_stride, sm_scale, dtype, B, H, N, D, dense,
                               dense_strides, work_counter, status, stream);
}

extern "C" int bsa_attn_bwd_dq(const void* q, const void* k, const void* v, const void* dout,
                               const int64_t strides[4], const float* lse2, const float* delta,
                               void* dq, const int32_t* row_ptr, const int32_t* col_idx,
                               int list_b_stride, int list_h_stride, float sm_scale, int dtype,
                               int B, int H, int N, int D, const uint8_t* dense,
                               const int64_t dense_strides[4], int32_t* work_counter,
                               int32_t* status, void* stream) {
  return bsa::launch_bwd<false>(q, k, v, dout, strides, lse2, delta, nullptr, dq, row_ptr,
                                col_idx, list_b_stride, list_h_stride, sm_scale, dtype, B, H, N,
                                D, dense, dense_strides, work_counter, status, stream);
}
