// Forward block-sparse attention for sm_100a.
//
// One CTA owns ONE query block (64 rows) of one (batch, head) and walks that block's list of key
// blocks two at a time ("supersteps").  The 64 query rows are loaded twice, as rows 0..63 and
// 64..127 of the tcgen05 A operand, so that the 128 TMEM lanes split the two key tiles of a
// superstep between them: lanes 0..63 own tile a, lanes 64..127 own tile b.  Every SM sub-partition
// (32 lanes) therefore always has the same amount of exp2 work, whatever the sparsity pattern —
// the exponentials, not the tensor pipe, bound this kernel at head dimension 64.
//   warp 8   : TMA producer — Q (twice) once, then only the listed K/V tiles into a 4-deep ring of
//              superstages (2 K tiles + 2 V tiles each)
//   warp 9   : S issuer and TMEM owner — S_u = [Q;Q] [K_a;K_b]^T as four M=128,N=128,K=16 MMAs into
//              one of 3 TMEM slots (lanes 0..63 use columns 0..63, lanes 64..127 columns 64..127;
//              an N=128 instruction occupies the tensor pipe no longer than an N=64 one)
//   warp 10  : P V issuer — O[g] += P_a[:, keys of group g] V_a[..] + P_b[:, keys of group g] V_b[..]
//              for key group g in {0, 1}: two accumulators, P read from TMEM, V an MN-major smem
//              operand.  Lanes 64..127 store zeros where tile a's P lives and lanes 0..63 where
//              tile b's does, so row r of an accumulator only ever sums tile-a products and row
//              r + 64 only tile-b products.  S and P V are issued by different warps so that
//              neither waits behind the other's barrier round trips.
//   warps 0..7 : online softmax.  Warp w works on TMEM lane quarter w % 4 and on key group
//              g = w / 4 (keys [32 g, +32) of its tile): tcgen05.ld of S, exp2, P written back over
//              the warp's own S columns as 16-bit, lazy rescale of its own accumulator.  The warps
//              never talk to each other inside the loop, so the two warps of a sub-partition
//              drift out of phase and overlap each other's exp2 and non-exp2 work.
// Each query row thus has four partial results (m, l, O) that the epilogue merges.
//
// Numerics follow the reference's loop (fa2_custom_mask/fa2_fwd.py:150-196): logits scaled by
// sm_scale*log2(e), exp2 domain, fp32 row sums of the fp32 probabilities, P rounded to the input
// dtype before P V.  The running maximum is only advanced when it grew by more than 8 (a factor
// 256), which leaves O = acc / l unchanged because both use the same reference maximum.
#include <math.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace bsa {

constexpr int kFwdStages = 4;   // superstages (2 K + 2 V tiles) in flight in shared memory
constexpr int kFwdSlots = 3;    // S/P supertiles (128 TMEM columns) in flight
constexpr int kFwdThreads = 352;
constexpr uint32_t kTileBytes = 64 * 64 * 2;       // one Q, K or V tile
constexpr uint32_t kFwdTmemCols = 512;
constexpr uint32_t kTmemO = 384;                   // O[g] at 384 + 64 g; slot r at 128 r
constexpr float kRescaleThreshold = 8.0f;
constexpr int kFwdMaxTiles = 2048;                 // key blocks per row that a CTA can list (N <= 131072)

struct FwdSmem {
  union {
    struct {
      uint8_t q[2][kTileBytes];                 // the query block, twice
      uint8_t k[kFwdStages][2][kTileBytes];
      uint8_t v[kFwdStages][2][kTileBytes];
    } t;
    float xfer[64][65];                         // epilogue: lanes 64..127 hand over, [col][row]
  } u;
  int32_t cols[kFwdMaxTiles];  // this query block's key-block list
  int wsum[kFwdThreads / 32];  // list building: kept blocks seen by each warp
  float mref[2][128];      // epilogue: reference maximum per key group and lane
  float lsum[2][128];      // epilogue: row sums
  float mtrue[2][128];     // epilogue: true running maxima
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];  // P V of the superstep done: stage free, S slot free, O updated
  uint64_t s_full[kFwdSlots];
  uint64_t p_full[kFwdSlots];
  uint32_t tmem_base;
  int abort_flag;
};

struct FwdParams {
  const int32_t* row_ptr;   // list mode: CSR row lists
  const int32_t* col_idx;
  const uint8_t* block;     // mask mode (block != nullptr): the CTA lists its own mask row
  int64_t ms0, ms1, ms2, ms3;
  void* o;
  int64_t o_sb, o_sh, o_sn;
  float* lse2;
  float* rowmax;
  int B, H, N, nb;
  int list_b_stride, list_h_stride;
  float scale_log2;
  int32_t* status;
};

enum FwdFail : int { kFailProducer = 1, kFailMma = 2, kFailSoftmax = 3 };

__device__ __forceinline__ void fwd_give_up(FwdSmem* sm, int32_t* status, int code) {
  sm->abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

// exp2 of one 32-column chunk of S against the row's reference maximum; returns the packed
// 16-bit probabilities and adds their fp32 sum to l.
template <bool kBf16>
__device__ __forceinline__ void exp_chunk(const uint32_t* sr, float c, float neg_m, uint32_t* pk,
                                          float& l) {
  float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float p0 = ex2_approx(fmaf(__uint_as_float(sr[i]), c, neg_m));
    const float p1 = ex2_approx(fmaf(__uint_as_float(sr[i + 1]), c, neg_m));
    const float p2 = ex2_approx(fmaf(__uint_as_float(sr[i + 2]), c, neg_m));
    const float p3 = ex2_approx(fmaf(__uint_as_float(sr[i + 3]), c, neg_m));
    l0 += p0;
    l1 += p1;
    l2 += p2;
    l3 += p3;
    pk[i / 2] = pack_2x16<kBf16>(p0, p1);
    pk[i / 2 + 1] = pack_2x16<kBf16>(p2, p3);
  }
  l += (l0 + l1) + (l2 + l3);
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

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;

  // ---- which query block ----
  const int bh = blockIdx.x / p.nb;
  const int mb = p.nb - 1 - (blockIdx.x % p.nb);  // late (long, if causal) rows first
  const int b = bh / p.H;
  const int h = bh % p.H;
  if (threadIdx.x == 0) BSA_TR(6, 0, 0);
  // ---- set-up; the Q load needs no list, so it starts first and overlaps the list building ----
  if (warp == 8 && lane == 0) {
#ifdef BSA_TRACE
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    BSA_TR_CTA(0, global_timer_ns());
    BSA_TR_CTA(2, smid);
#endif
    mbar_init(smem_u32(&sm->q_full), 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm->kv_full[s]), 1);
      mbar_init(smem_u32(&sm->kv_empty[s]), 1);
    }
    for (int i = 0; i < kFwdSlots; ++i) {
      mbar_init(smem_u32(&sm->s_full[i]), 1);
      mbar_init(smem_u32(&sm->p_full[i]), 8);  // one arrival per softmax warp
    }
    sm->abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    const uint32_t bar = smem_u32(&sm->q_full);
    mbar_expect_tx(bar, 2 * kTileBytes);
    tma_load_4d(smem_u32(sm->u.t.q[0]), &tm_q, bar, 0, mb * 64, h, b);
    tma_load_4d(smem_u32(sm->u.t.q[1]), &tm_q, bar, 0, mb * 64, h, b);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }

  // ---- this query block's key-block list, into shared memory ----
  int n_tiles = 0;
  if (p.block != nullptr) {
    // mask mode: ordered compaction of the kept blocks of mask row (b, h, mb); list_*_stride are
    // 0 for a broadcast axis and 1 otherwise here
    const uint8_t* mrow = p.block + (b * p.list_b_stride) * p.ms0 + (h * p.list_h_stride) * p.ms1 +
                          static_cast<int64_t>(mb) * p.ms2;
    for (int c0 = 0; c0 < p.nb; c0 += kFwdThreads) {
      const int c = c0 + static_cast<int>(threadIdx.x);
      const bool keep = c < p.nb && mrow[c * p.ms3] != 0;
      const unsigned bal = __ballot_sync(0xffffffffu, keep);
      if (lane == 0) sm->wsum[warp] = __popc(bal);
      __syncthreads();
      int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kFwdThreads / 32; ++w) {
        const int cnt = sm->wsum[w];
        before += w < warp ? cnt : 0;
        total += cnt;
      }
      if (keep) sm->cols[n_tiles + before + __popc(bal & ((1u << lane) - 1u))] = c;
      n_tiles += total;
      __syncthreads();
    }
  } else {
    const int64_t li = static_cast<int64_t>(b * p.list_b_stride + h * p.list_h_stride) * p.nb + mb;
    const int beg = __ldg(p.row_ptr + li);
    n_tiles = __ldg(p.row_ptr + li + 1) - beg;
    for (int i = threadIdx.x; i < n_tiles; i += kFwdThreads) sm->cols[i] = __ldg(p.col_idx + beg + i);
  }
  const int n_super = (n_tiles + 1) >> 1;
  const int32_t* cols = sm->cols;  // visible to every role after the set-up barrier
  if (threadIdx.x == 0) BSA_TR(6, 0, 1);
  if (threadIdx.x == 0) BSA_TR_CTA(3, n_tiles);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->abort_flag;
  if (threadIdx.x == 0) BSA_TR(6, 0, 2);

  if (warp == 8) {
    // =========================== TMA producer ===========================
    if (n_super == 0) {
      // nobody consumes Q then, but its copy must have landed before shared memory is given back
      if (!mbar_wait_warp(smem_u32(&sm->q_full), 0, abort_flag))
        fwd_give_up(sm, p.status, kFailProducer);
    } else {
      const bool leader = elect_one();
      for (int u = 0; u < n_super; ++u) {
        const int ss = u % kFwdStages;
        const int nt = min(2, n_tiles - 2 * u);
        const int n0 = cols[2 * u];
        const int n1 = nt == 2 ? cols[2 * u + 1] : 0;
        if (!mbar_wait_warp(smem_u32(&sm->kv_empty[ss]), ((u / kFwdStages) & 1) ^ 1, abort_flag)) {
          fwd_give_up(sm, p.status, kFailProducer);
          break;
        }
        if (leader) {
          BSA_TR(0, u, 0);
          const uint32_t bar = smem_u32(&sm->kv_full[ss]);
          mbar_expect_tx(bar, 2 * kTileBytes * nt);
          tma_load_4d(smem_u32(sm->u.t.k[ss][0]), &tm_k, bar, 0, n0 * 64, h, b);
          tma_load_4d(smem_u32(sm->u.t.v[ss][0]), &tm_v, bar, 0, n0 * 64, h, b);
          if (nt == 2) {
            tma_load_4d(smem_u32(sm->u.t.k[ss][1]), &tm_k, bar, 0, n1 * 64, h, b);
            tma_load_4d(smem_u32(sm->u.t.v[ss][1]), &tm_v, bar, 0, n1 * 64, h, b);
          }
          BSA_TR(0, u, 1);
        }
      }
    }
  } else if (warp == 9) {
    // =========================== S issuer ===========================
    if (n_super > 0) {
      constexpr uint32_t idesc_s128 = umma_idesc(kBf16, 0, 0, 128, 128);  // [Q;Q] x [K_a;K_b]
      constexpr uint32_t idesc_s64 = umma_idesc(kBf16, 0, 0, 128, 64);    // odd tail: one tile
      const bool leader = elect_one();
      const uint64_t desc_q = smem_desc_sw128(smem_u32(sm->u.t.q[0]), 16, 1024);
      const uint64_t desc_k0 = smem_desc_sw128(smem_u32(sm->u.t.k[0][0]), 16, 1024);
      bool ok = mbar_wait_warp(smem_u32(&sm->q_full), 0, abort_flag);
      for (int u = 0; ok && u < n_super; ++u) {
        const int ss = u % kFwdStages;
        const int slot = u % kFwdSlots;
        const int nt = min(2, n_tiles - 2 * u);
        ok = mbar_wait_warp(smem_u32(&sm->kv_full[ss]), (u / kFwdStages) & 1, abort_flag);
        if (!ok) break;
        if (u >= kFwdSlots) {
          // the slot still holds P of superstep u-3 until that superstep's P V is complete
          const int up = u - kFwdSlots;
          ok = mbar_wait_warp(smem_u32(&sm->kv_empty[up % kFwdStages]), (up / kFwdStages) & 1,
                              abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        if (leader) {
          BSA_TR(1, u, 0);
          const uint64_t desc_k = desc_k0 + static_cast<uint64_t>(ss * ((2 * kTileBytes) >> 4));
          const uint32_t idesc = nt == 2 ? idesc_s128 : idesc_s64;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + 128 * slot, desc_q + 2 * kk, desc_k + 2 * kk, idesc, kk > 0);
          tc_commit(smem_u32(&sm->s_full[slot]));
          BSA_TR(1, u, 1);
        }
      }
      if (!ok) fwd_give_up(sm, p.status, kFailMma);
    }
  } else if (warp == 10) {
    // =========================== P V issuer ===========================
    if (n_super > 0) {
      constexpr uint32_t idesc_pv = umma_idesc(kBf16, 0, 1, 128, 64);  // P (TMEM) x V (MN-major)
      const bool leader = elect_one();
      const uint64_t desc_v0 = smem_desc_sw128(smem_u32(sm->u.t.v[0][0]), 8192, 1024);
      bool ok = true;
      for (int u = 0; ok && u < n_super; ++u) {
        const int ss = u % kFwdStages;
        const int slot = u % kFwdSlots;
        const int nt = min(2, n_tiles - 2 * u);
        ok = mbar_wait_warp(smem_u32(&sm->p_full[slot]), (u / kFwdSlots) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          BSA_TR(7, u, 0);
          // P of tile t sits over that tile's own S columns: keys [32 g + 16 k2, +16) of tile t at
          // slot column 64 t + 32 g + 8 k2; the other half of the lanes holds zeros there
          for (int g = 0; g < 2; ++g) {
            for (int t = 0; t < nt; ++t) {
              const uint64_t desc_v =
                  desc_v0 + static_cast<uint64_t>((ss * 2 + t) * (kTileBytes >> 4));
#pragma unroll
              for (int k2 = 0; k2 < 2; ++k2)
                umma_ts(tmem + kTmemO + 64 * g, tmem + 128 * slot + 64 * t + 32 * g + 8 * k2,
                        desc_v + 128 * (2 * g + k2), idesc_pv, (u > 0) || (t > 0) || (k2 > 0));
            }
          }
          tc_commit(smem_u32(&sm->kv_empty[ss]));
          BSA_TR(7, u, 1);
        }
      }
      if (!ok) fwd_give_up(sm, p.status, kFailMma);
    }
  } else {
    // =========================== softmax + epilogue ===========================
    const int g = warp >> 2;          // key columns [32 g, +32) of the tile
    const int quarter = warp & 3;     // TMEM lane quarter this warp may touch
    const int t_mine = quarter >> 1;  // lanes 0..63 own tile a of a superstep, 64..127 tile b
    const int lane_row = quarter * 32 + lane;          // TMEM lane
    const int r_blk = (quarter & 1) * 32 + lane;       // row of the query block
    const int row = mb * 64 + r_blk;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem + lane_base + kTmemO + 64 * g;
    const float c = p.scale_log2;
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;

    for (int u = 0; u < n_super; ++u) {
      const int slot = u % kFwdSlots;
      const int nt = min(2, n_tiles - 2 * u);
      ok = mbar_wait_warp(smem_u32(&sm->s_full[slot]), (u / kFwdSlots) & 1, abort_flag);
      if (!ok) break;
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 0);
      if (1 - t_mine < nt) {
        // the other tile's P V also sweeps these lanes: give it zeros where that tile's P lives
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) z[i] = 0u;
        tc_fence_after();
        tmem_st_32x32b_x16(tmem + lane_base + 128 * slot + 64 * (1 - t_mine) + 32 * g, z);
        if (t_mine >= nt) {
          tc_wait_st();
          tc_fence_before();
        }
      }
      if (t_mine < nt) {
        tc_fence_after();
        // this warp's S: columns [64 t + 32 g, +32) of the slot; its P goes over the first 16
        const uint32_t s_addr = tmem + lane_base + 128 * slot + 64 * t_mine + 32 * g;
        uint32_t sr[32], pk[16];
        tmem_ld_32x32b_x32(s_addr, sr);
        tc_wait_ld();
        if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 1);
        const float zmax = max_chunk(sr) * c;
        m_true = fmaxf(m_true, zmax);
        float alpha = 1.f;
        bool rescale = false;
        if (m_ref == -INFINITY) {
          m_ref = zmax;  // first tile of this lane: O and l are still zero
        } else if (zmax > m_ref + kRescaleThreshold) {
          alpha = ex2_approx(m_ref - zmax);
          l *= alpha;
          m_ref = zmax;
          rescale = true;
        }
        if (__any_sync(0xffffffffu, rescale)) {
          // This warp's O must hold the previous superstep's product (u >= 1 here) first: P V of
          // superstep u-1 completing frees that superstep's stage.  S_u being complete implies
          // P V of u-3 and earlier are complete, and P V of u+3 cannot complete before this warp
          // delivers P_u, so the awaited phase is unambiguous.
          ok = mbar_wait_warp(smem_u32(&sm->kv_empty[(u - 1) % kFwdStages]),
                              ((u - 1) / kFwdStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            uint32_t orow[32];
            tmem_ld_32x32b_x32(o_addr + 32 * part, orow);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
            tmem_st_32x32b_x32(o_addr + 32 * part, orow);
          }
        }
        exp_chunk<kBf16>(sr, c, -m_ref, pk, l);
        if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 2);
        tmem_st_32x32b_x16(s_addr, pk);
        tc_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[slot]));
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 3);
    }

    // ---- epilogue: merge the four partial results of every query row ----
    // (key groups 0/1 x lanes r / r + 64).  A warp reads both accumulators of its own lanes
    // straight from TMEM; only the hand-over from lanes 64..127 to lanes 0..63 goes through
    // shared memory (the K/V ring, dead once the last P V is complete).
    if (ok && n_super > 0)
      ok = mbar_wait_warp(smem_u32(&sm->kv_empty[(n_super - 1) % kFwdStages]),
                          ((n_super - 1) / kFwdStages) & 1, abort_flag);
    if (!ok) fwd_give_up(sm, p.status, kFailSoftmax);
    if (threadIdx.x == 0) BSA_TR(6, 1, 0);
    sm->mref[g][lane_row] = m_ref;
    sm->lsum[g][lane_row] = l;
    sm->mtrue[g][lane_row] = m_true;
    named_barrier_sync(1, 256);  // every softmax warp arrives at each of these, also after a give-up
    const bool live = !*abort_flag;
    if (threadIdx.x == 0) BSA_TR(6, 1, 1);
    float m_all = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) m_all = fmaxf(m_all, sm->mref[i & 1][r_blk + 64 * (i >> 1)]);
    float l_all = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float mi = sm->mref[i & 1][r_blk + 64 * (i >> 1)];
      if (mi != -INFINITY) l_all += ex2_approx(mi - m_all) * sm->lsum[i & 1][r_blk + 64 * (i >> 1)];
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    // weights of this lane's two accumulator rows; this warp merges columns [32 g, +32) of both
    const float m0 = sm->mref[0][lane_row], m1 = sm->mref[1][lane_row];
    const float w0 = m0 == -INFINITY ? 0.f : ex2_approx(m0 - m_all) * inv;
    const float w1 = m1 == -INFINITY ? 0.f : ex2_approx(m1 - m_all) * inv;
    float acc[32];
    if (live && n_super > 0) {  // warp-uniform
      uint32_t a0[32], a1[32];
      tc_fence_after();
      tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 32 * g, a0);
      tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 64 + 32 * g, a1);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        acc[i] = fmaf(__uint_as_float(a1[i]), w1, __uint_as_float(a0[i]) * w0);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    }
    if (t_mine == 1) {
#pragma unroll
      for (int i = 0; i < 32; ++i) sm->u.xfer[32 * g + i][r_blk] = acc[i];
    }
    named_barrier_sync(1, 256);
    if (threadIdx.x == 0) BSA_TR(6, 1, 2);
    if (t_mine == 0 && live) {
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2)
        packed[i / 2] = pack_2x16<kBf16>(acc[i] + sm->u.xfer[32 * g + i][r_blk],
                                         acc[i + 1] + sm->u.xfer[32 * g + i + 1][r_blk]);
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o) + b * p.o_sb + h * p.o_sh +
                                            static_cast<int64_t>(row) * p.o_sn + 32 * g);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      if (g == 0) {
        const int64_t ri = (static_cast<int64_t>(b) * p.H + h) * p.N + row;
        p.lse2[ri] = l_all > 0.f ? m_all + lg2_approx(l_all) : -INFINITY;
        if (p.rowmax)
          p.rowmax[ri] = fmaxf(fmaxf(sm->mtrue[0][r_blk], sm->mtrue[1][r_blk]),
                               fmaxf(sm->mtrue[0][r_blk + 64], sm->mtrue[1][r_blk + 64]));
      }
    }
    if (threadIdx.x == 0) BSA_TR(6, 1, 3);
  }

  // ---- tear-down: every role arrives here, also after a give-up ----
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
  if (threadIdx.x == 0) BSA_TR(6, 2, 0);
  if (threadIdx.x == 0) BSA_TR_CTA(1, global_timer_ns());
}

}  // namespace bsa

#ifdef BSA_TRACE
extern "C" int bsa_debug_copy_cta_times(unsigned long long* host) {
  return cudaMemcpyFromSymbol(host, bsa::g_bsa_cta_times, sizeof(bsa::g_bsa_cta_times)) == cudaSuccess ? 0 : -5;
}
extern "C" int bsa_debug_copy_trace(long long* host) {
  return cudaMemcpyFromSymbol(host, bsa::g_bsa_trace, sizeof(bsa::g_bsa_trace)) == cudaSuccess ? 0 : -5;
}
#endif

namespace bsa {

static int launch_fwd(const void* q, const int64_t q_strides[4], const void* k,
                      const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* o,
                      const int64_t o_strides[4], float* lse2, float* rowmax,
                      const int32_t* row_ptr, const int32_t* col_idx, const uint8_t* block,
                      const int64_t* block_strides, int list_b_stride, int list_h_stride,
                      float sm_scale, int dtype, int B, int H, int N, int D, int32_t* status,
                      void* stream) {
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!lse2 || (block == nullptr && (!row_ptr || !col_idx))) return BSA_ERR_BAD_POINTER;
  int rc;
  if ((rc = check_qkv_operand(q, q_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(k, k_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(v, v_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(o, o_strides)) != BSA_OK) return rc;
  if ((rc = check_device_sm100()) != BSA_OK) return rc;

  const int nb = N / kBlock;
  if (nb > kFwdMaxTiles) return BSA_ERR_TOO_LARGE;
  if (static_cast<int64_t>(B) * H * nb > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = make_qkv_tmap(&tm_q, q, q_strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_k, k, k_strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_v, v, v_strides, B, H, N, dtype, 64)) != BSA_OK) return rc;

  FwdParams prm;
  prm.row_ptr = row_ptr;
  prm.col_idx = col_idx;
  prm.block = block;
  prm.ms0 = block ? block_strides[0] : 0;
  prm.ms1 = block ? block_strides[1] : 0;
  prm.ms2 = block ? block_strides[2] : 0;
  prm.ms3 = block ? block_strides[3] : 0;
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
  prm.list_b_stride = list_b_stride;
  prm.list_h_stride = list_h_stride;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.status = status;

  const size_t smem_bytes = sizeof(FwdSmem) + 1024;
  auto kern = dtype == BSA_BF16 ? attn_fwd_kernel<true> : attn_fwd_kernel<false>;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) != BSA_OK)
    return rc;
  const dim3 grid(static_cast<unsigned>(B * H * nb));
  kern<<<grid, kFwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, prm);
  if (cudaGetLastError() != cudaSuccess) return BSA_ERR_CUDA;
  return BSA_OK;
}

}  // namespace bsa

extern "C" int bsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k,
                            const int64_t k_strides[4], const void* v, const int64_t v_strides[4],
                            void* o, const int64_t o_strides[4], float* lse2, float* rowmax,
                            const int32_t* row_ptr, const int32_t* col_idx, int list_b_stride,
                            int list_h_stride, float sm_scale, int dtype, int B, int H, int N,
                            int D, int32_t* status, void* stream) {
  if (!row_ptr || !col_idx) return BSA_ERR_BAD_POINTER;
  return bsa::launch_fwd(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, rowmax,
                         row_ptr, col_idx, nullptr, nullptr, list_b_stride, list_h_stride, sm_scale,
                         dtype, B, H, N, D, status, stream);
}

extern "C" int bsa_attn_fwd_block_mask(const void* q, const int64_t q_strides[4], const void* k,
                                       const int64_t k_strides[4], const void* v,
                                       const int64_t v_strides[4], void* o,
                                       const int64_t o_strides[4], float* lse2, float* rowmax,
                                       const uint8_t* block, const int64_t block_strides[4],
                                       int Bm, int Hm, float sm_scale, int dtype, int B, int H,
                                       int N, int D, int32_t* status, void* stream) {
  if (!block || !block_strides) return BSA_ERR_BAD_POINTER;
  if ((Bm != 1 && Bm != B) || (Hm != 1 && Hm != H)) return BSA_ERR_BAD_SHAPE;
  for (int i = 0; i < 4; ++i)
    if (block_strides[i] < 0) return BSA_ERR_BAD_STRIDE;
  return bsa::launch_fwd(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, rowmax,
                         nullptr, nullptr, block, block_strides, Bm > 1 ? 1 : 0, Hm > 1 ? 1 : 0,
                         sm_scale, dtype, B, H, N, D, status, stream);
}
