// Forward block-sparse attention for sm_100a.
//
// One CTA owns one PAIR of adjacent query blocks (128 query rows = the 128 lanes of a tcgen05
// accumulator) of one (batch, head) and walks that pair's list of key blocks two at a time
// ("supersteps" of up to 128 keys):
//   warp 8   : TMA producer — Q once, then only the listed K/V tiles into a 4-deep ring of
//              superstages (2 K tiles + 2 V tiles each)
//   warp 9   : S issuer and TMEM owner — S_u = Q [K_a;K_b]^T as four M=128,N=128,K=16 MMAs into a
//              ring of 3 TMEM slots (an N=128 instruction keeps the tensor pipe at full rate; an
//              N=64 one occupies it just as long)
//   warp 10  : P V issuer — O_g += P_u[:, keys of group g] V[keys of group g] with P read from
//              TMEM and V as an MN-major smem operand.  S and P V are issued by different warps so
//              that neither waits behind the other's barrier round trips.
//   warps 0..3 (group 0: keys 0..31 of every tile) and 4..7 (group 1: keys 32..63): online
//              softmax, one thread per query row (TMEM lane) and group: tcgen05.ld of S, exp2, P
//              written back over the group's own S columns as 16-bit, lazy rescale of the group's
//              own O.  The groups never talk to each other during the loop: each keeps its own
//              running maximum, row sum and accumulator, and every SM sub-partition always has
//              two equally loaded softmax warps.
// The two partial results (m, l, O) of a row are merged in the epilogue.
// A key block listed by only one of the two query blocks still runs as M=128 MMAs; the warps of
// the other half store P = 0 for it and skip the exponentials.
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
constexpr uint32_t kTileBytes = 64 * 64 * 2;       // one K or V tile
constexpr uint32_t kQBytes = 128 * 64 * 2;         // one query-pair tile
constexpr uint32_t kFwdTmemCols = 512;
constexpr uint32_t kTmemO = 384;                   // O of group g at kTmemO + 64 g; slot r at 128 r
constexpr float kRescaleThreshold = 8.0f;

struct FwdSmem {
  uint8_t q[kQBytes];
  uint8_t k[kFwdStages][2][kTileBytes];
  uint8_t v[kFwdStages][2][kTileBytes];
  float stats[2][128][2];  // (m_ref, l) of every row, per softmax group, for the final merge
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];  // P V of the superstep done: stage free, S slot free, O updated
  uint64_t s_full[kFwdSlots];
  uint64_t p_full[kFwdSlots];
  uint32_t tmem_base;
  int abort_flag;
};

struct FwdParams {
  const int32_t* pair_ptr;
  const int32_t* pair_ent;
  void* o;
  int64_t o_sb, o_sh, o_sn;
  float* lse2;
  float* rowmax;
  int B, H, N, npair;
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

__device__ __forceinline__ float max_chunk(const uint32_t* sr) {
  float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]);
  float mx2 = __uint_as_float(sr[2]), mx3 = __uint_as_float(sr[3]);
#pragma unroll
  for (int i = 4; i < 32; i += 4) {
    mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
    mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
    mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
    mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
  }
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
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

  // ---- which query pair ----
  const int bh = blockIdx.x / p.npair;
  const int pr = p.npair - 1 - (blockIdx.x % p.npair);  // late (long, if causal) pairs first
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int64_t li = static_cast<int64_t>(b * p.list_b_stride + h * p.list_h_stride) * p.npair + pr;
  const int beg = __ldg(p.pair_ptr + li);
  const int n_tiles = __ldg(p.pair_ptr + li + 1) - beg;
  const int n_super = (n_tiles + 1) >> 1;
  const int32_t* ents = p.pair_ent + beg;

  // ---- set-up ----
  if (threadIdx.x == 0) {
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
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->abort_flag;

  if (warp == 8) {
    // =========================== TMA producer ===========================
    if (n_super > 0) {
      const bool leader = elect_one();
      if (leader) {
        mbar_expect_tx(smem_u32(&sm->q_full), kQBytes);
        tma_load_4d(smem_u32(sm->q), &tm_q, smem_u32(&sm->q_full), 0, pr * 128, h, b);
      }
      for (int u = 0; u < n_super; ++u) {
        const int ss = u % kFwdStages;
        const int nt = min(2, n_tiles - 2 * u);
        const int n0 = __ldg(ents + 2 * u) >> 2;
        const int n1 = nt == 2 ? (__ldg(ents + 2 * u + 1) >> 2) : 0;
        if (!mbar_wait_warp(smem_u32(&sm->kv_empty[ss]), ((u / kFwdStages) & 1) ^ 1, abort_flag)) {
          fwd_give_up(sm, p.status, kFailProducer);
          break;
        }
        if (leader) {
          BSA_TR(0, u, 0);
          const uint32_t bar = smem_u32(&sm->kv_full[ss]);
          mbar_expect_tx(bar, 2 * kTileBytes * nt);
          tma_load_4d(smem_u32(sm->k[ss][0]), &tm_k, bar, 0, n0 * 64, h, b);
          tma_load_4d(smem_u32(sm->v[ss][0]), &tm_v, bar, 0, n0 * 64, h, b);
          if (nt == 2) {
            tma_load_4d(smem_u32(sm->k[ss][1]), &tm_k, bar, 0, n1 * 64, h, b);
            tma_load_4d(smem_u32(sm->v[ss][1]), &tm_v, bar, 0, n1 * 64, h, b);
          }
          BSA_TR(0, u, 1);
        }
      }
    }
  } else if (warp == 9) {
    // =========================== S issuer ===========================
    if (n_super > 0) {
      constexpr uint32_t idesc_s128 = umma_idesc(kBf16, 0, 0, 128, 128);  // Q x [K_a;K_b]
      constexpr uint32_t idesc_s64 = umma_idesc(kBf16, 0, 0, 128, 64);    // odd tail: one tile
      const bool leader = elect_one();
      const uint64_t desc_q = smem_desc_sw128(smem_u32(sm->q), 16, 1024);
      const uint64_t desc_k0 = smem_desc_sw128(smem_u32(sm->k[0][0]), 16, 1024);
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
      const uint64_t desc_v0 = smem_desc_sw128(smem_u32(sm->v[0][0]), 8192, 1024);
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
          // P of the slot: columns [32 g + 16 t, +16) hold keys [32 g, 32 g + 32) of tile t
          for (int g = 0; g < 2; ++g) {
            const uint32_t d_o = tmem + kTmemO + 64 * g;
            for (int t = 0; t < nt; ++t) {
              const uint64_t desc_v =
                  desc_v0 + static_cast<uint64_t>((ss * 2 + t) * (kTileBytes >> 4));
#pragma unroll
              for (int k2 = 0; k2 < 2; ++k2)
                umma_ts(d_o, tmem + 128 * slot + 32 * g + 16 * t + 8 * k2,
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
    const int g = warp >> 2;          // softmax group: keys [32 g, 32 g + 32) of every tile
    const int quarter = warp & 3;     // TMEM lane quarter this warp may touch
    const int half = quarter >> 1;    // which query block of the pair
    const int r_cta = quarter * 32 + lane;
    const int row = pr * 128 + r_cta;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem + lane_base + kTmemO + 64 * g;
    const float c = p.scale_log2;
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    int e0 = n_tiles > 0 ? __ldg(ents) : 0;
    int e1 = n_tiles > 1 ? __ldg(ents + 1) : 0;

    for (int u = 0; u < n_super; ++u) {
      const int slot = u % kFwdSlots;
      const int nt = min(2, n_tiles - 2 * u);
      const bool listed0 = ((e0 >> half) & 1) != 0;
      const bool listed1 = nt == 2 && ((e1 >> half) & 1) != 0;
      if (2 * u + 2 < n_tiles) e0 = __ldg(ents + 2 * u + 2);
      if (2 * u + 3 < n_tiles) e1 = __ldg(ents + 2 * u + 3);
      ok = mbar_wait_warp(smem_u32(&sm->s_full[slot]), (u / kFwdSlots) & 1, abort_flag);
      if (!ok) break;
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 0);
      tc_fence_after();
      // S of tile t, this group's keys: columns [64 t + 32 g, +32) of the slot; the group's P goes
      // over its own tile-a columns: [32 g + 16 t, +16)
      const uint32_t s_addr = tmem + lane_base + 128 * slot + 32 * g;
      uint32_t pk0[16], pk1[16];
      if (listed0 || listed1) {
        uint32_t sr0[32], sr1[32];
        if (listed0) tmem_ld_32x32b_x32(s_addr, sr0);
        if (listed1) tmem_ld_32x32b_x32(s_addr + 64, sr1);
        tc_wait_ld();
        if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 1);
        float mx = -INFINITY;
        if (listed0) mx = max_chunk(sr0);
        if (listed1) mx = fmaxf(mx, max_chunk(sr1));
        const float zmax = mx * c;
        m_true = fmaxf(m_true, zmax);
        float alpha = 1.f;
        bool rescale = false;
        if (m_ref == -INFINITY) {
          m_ref = zmax;  // first listed tile of this row in this group: O and l are still zero
        } else if (zmax > m_ref + kRescaleThreshold) {
          alpha = ex2_approx(m_ref - zmax);
          l *= alpha;
          m_ref = zmax;
          rescale = true;
        }
        if (__any_sync(0xffffffffu, rescale)) {
          // The group's O must hold the previous superstep's product (u >= 1 here) before it is
          // scaled.  P V of superstep u-1 completing frees that superstep's stage; S_u being
          // complete implies P V of u-3 and earlier are complete, and P V of u+3 cannot complete
          // before this warp delivers P_u, so the awaited phase is unambiguous.
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
        const float neg_m = -m_ref;
        if (listed0) {
          exp_chunk<kBf16>(sr0, c, neg_m, pk0, l);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk0[i] = 0u;
        }
        if (listed1) {
          exp_chunk<kBf16>(sr1, c, neg_m, pk1, l);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk1[i] = 0u;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk0[i] = 0u;
          pk1[i] = 0u;
        }
      }
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 2);
      tmem_st_32x32b_x16(s_addr, pk0);
      if (nt == 2) tmem_st_32x32b_x16(s_addr + 16, pk1);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[slot]));
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), u, 3);
    }

    // ---- epilogue: merge the two groups' partial results of every row ----
    // The last P V frees the last stage; every earlier phase of that barrier is long complete.
    if (ok && n_super > 0)
      ok = mbar_wait_warp(smem_u32(&sm->kv_empty[(n_super - 1) % kFwdStages]),
                          ((n_super - 1) / kFwdStages) & 1, abort_flag);
    if (!ok) fwd_give_up(sm, p.status, kFailSoftmax);
    sm->stats[g][r_cta][0] = m_ref;
    sm->stats[g][r_cta][1] = l;
    named_barrier_sync(1, 256);  // every softmax warp arrives exactly once, also after a give-up
    const bool live = !*abort_flag;
    const float m_o = sm->stats[g ^ 1][r_cta][0];
    const float l_o = sm->stats[g ^ 1][r_cta][1];
    if (p.rowmax) {
      // the true running maximum goes through the same smem words once everyone has read them
      named_barrier_sync(2, 256);
      sm->stats[g][r_cta][0] = m_true;
      named_barrier_sync(2, 256);
      if (live && g == 0 && row < p.N)
        p.rowmax[(static_cast<int64_t>(b) * p.H + h) * p.N + row] =
            fmaxf(m_true, sm->stats[1][r_cta][0]);
    }
    if (live) {
      const float m_all = fmaxf(m_ref, m_o);
      const float w_me = m_ref == -INFINITY ? 0.f : ex2_approx(m_ref - m_all);
      const float w_ot = m_o == -INFINITY ? 0.f : ex2_approx(m_o - m_all);
      const float l_all = w_me * l + w_ot * l_o;
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      // weights of accumulator 0 / 1 (both are written by every superstep)
      const float w0 = (g == 0 ? w_me : w_ot) * inv;
      const float w1 = (g == 0 ? w_ot : w_me) * inv;
      uint32_t packed[16];
      if (n_super > 0) {
        tc_fence_after();
        uint32_t a0[32], a1[32];
        tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 32 * g, a0);
        tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 64 + 32 * g, a1);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = __uint_as_float(a0[i]) * w0, x1 = __uint_as_float(a0[i + 1]) * w0;
          x0 = fmaf(__uint_as_float(a1[i]), w1, x0);
          x1 = fmaf(__uint_as_float(a1[i + 1]), w1, x1);
          packed[i / 2] = pack_2x16<kBf16>(x0, x1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = 0u;
      }
      if (row < p.N) {
        // group g writes columns [32 g, 32 g + 32) of the row
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o) + b * p.o_sb +
                                              h * p.o_sh + static_cast<int64_t>(row) * p.o_sn +
                                              32 * g);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2],
                              packed[4 * i + 3]);
        if (g == 0) {
          const int64_t ri = (static_cast<int64_t>(b) * p.H + h) * p.N + row;
          p.lse2[ri] = l_all > 0.f ? m_all + lg2_approx(l_all) : -INFINITY;
        }
      }
    }
  }

  // ---- tear-down: every role arrives here, also after a give-up ----
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

}  // namespace bsa

#ifdef BSA_TRACE
extern "C" int bsa_debug_copy_trace(long long* host) {
  return cudaMemcpyFromSymbol(host, bsa::g_bsa_trace, sizeof(bsa::g_bsa_trace)) == cudaSuccess ? 0 : -5;
}
#endif

extern "C" int bsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k,
                            const int64_t k_strides[4], const void* v, const int64_t v_strides[4],
                            void* o, const int64_t o_strides[4], float* lse2, float* rowmax,
                            const int32_t* qpair_ptr, const int32_t* qpair_ent, int list_b_stride,
                            int list_h_stride, float sm_scale, int dtype, int B, int H, int N,
                            int D, int32_t* status, void* stream) {
  using namespace bsa;
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!lse2 || !qpair_ptr || !qpair_ent) return BSA_ERR_BAD_POINTER;
  int rc;
  if ((rc = check_qkv_operand(q, q_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(k, k_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(v, v_strides)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(o, o_strides)) != BSA_OK) return rc;
  if ((rc = check_device_sm100()) != BSA_OK) return rc;

  const int nb = N / kBlock;
  const int npair = (nb + 1) / 2;
  if (static_cast<int64_t>(B) * H * npair > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = make_qkv_tmap(&tm_q, q, q_strides, B, H, N, dtype, 128)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_k, k, k_strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_v, v, v_strides, B, H, N, dtype, 64)) != BSA_OK) return rc;

  FwdParams prm;
  prm.pair_ptr = qpair_ptr;
  prm.pair_ent = qpair_ent;
  prm.o = o;
  prm.o_sb = o_strides[0];
  prm.o_sh = o_strides[1];
  prm.o_sn = o_strides[2];
  prm.lse2 = lse2;
  prm.rowmax = rowmax;
  prm.B = B;
  prm.H = H;
  prm.N = N;
  prm.npair = npair;
  prm.list_b_stride = list_b_stride;
  prm.list_h_stride = list_h_stride;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.status = status;

  const size_t smem_bytes = sizeof(FwdSmem) + 1024;
  auto kern = dtype == BSA_BF16 ? attn_fwd_kernel<true> : attn_fwd_kernel<false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem_bytes)) != cudaSuccess) {
    (void)cudaGetLastError();
    return BSA_ERR_CUDA;
  }
  const dim3 grid(static_cast<unsigned>(B * H * npair));
  kern<<<grid, kFwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, prm);
  if (cudaGetLastError() != cudaSuccess) return BSA_ERR_CUDA;
  return BSA_OK;
}
