// Forward block-sparse attention for sm_100a.
//
// One CTA owns one PAIR of adjacent query blocks (128 query rows = the 128 lanes of a tcgen05
// accumulator) of one (batch, head) and walks that pair's list of key blocks ("steps"):
//   warp 8  : TMA producer — Q once, then only the listed K/V tiles into an 8-stage smem ring
//   warp 9  : tcgen05.mma issuer and TMEM owner — S_j = Q K_j^T into a ring of 4 TMEM slots, issued
//             up to 4 steps ahead; O_g += P_j V_j with P read from TMEM and V as an MN-major
//             smem operand, into the accumulator of softmax group g = j mod 2
//   warps 0..3 (group 0, even steps) and 4..7 (group 1, odd steps): online softmax, one thread
//             per query row (TMEM lane): tcgen05.ld of S, exp2, P written back over S as 16-bit,
//             lazy rescale of the group's own O.  Two groups give every SM sub-partition two
//             softmax warps to interleave, and let the two halves of the pair drift apart.
// The two partial results (m, l, O) of a row are merged in the epilogue.
// A key block listed by only one of the two query blocks still runs as an M=128 MMA; the warps of
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

constexpr int kFwdStages = 8;   // K/V tiles in flight in shared memory
constexpr int kFwdSlots = 4;    // S/P tiles in flight in TMEM
constexpr int kFwdThreads = 320;
constexpr uint32_t kTileBytes = 64 * 64 * 2;       // one K or V tile
constexpr uint32_t kQBytes = 128 * 64 * 2;         // one query-pair tile
constexpr uint32_t kFwdTmemCols = 512;
constexpr uint32_t kTmemO = 256;                   // O of group g at kTmemO + 64 g; slot r at 64 r
constexpr float kRescaleThreshold = 8.0f;

struct FwdSmem {
  uint8_t q[kQBytes];
  uint8_t k[kFwdStages][kTileBytes];
  uint8_t v[kFwdStages][kTileBytes];
  float stats[2][128][2];  // (m_ref, l) of every row, per softmax group, for the final merge
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
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
  const int n_steps = __ldg(p.pair_ptr + li + 1) - beg;
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
      mbar_init(smem_u32(&sm->p_full[i]), 4);  // one arrival per warp of the step's group
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
    if (n_steps > 0) {
      const bool leader = elect_one();
      if (leader) {
        mbar_expect_tx(smem_u32(&sm->q_full), kQBytes);
        tma_load_4d(smem_u32(sm->q), &tm_q, smem_u32(&sm->q_full), 0, pr * 128, h, b);
      }
      for (int j = 0; j < n_steps; ++j) {
        const int s = j % kFwdStages;
        const uint32_t ph = (j / kFwdStages) & 1;
        if (!mbar_wait_warp(smem_u32(&sm->kv_empty[s]), ph ^ 1, abort_flag)) {
          fwd_give_up(sm, p.status, kFailProducer);
          break;
        }
        if (lane == 0) BSA_TR(0, j, 0);
        const int nblk = __ldg(ents + j) >> 2;
        if (leader) {
          const uint32_t bar = smem_u32(&sm->kv_full[s]);
          mbar_expect_tx(bar, 2 * kTileBytes);
          tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, nblk * 64, h, b);
          tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, nblk * 64, h, b);
          BSA_TR(0, j, 1);
        }
      }
    }
  } else if (warp == 9) {
    // =========================== MMA issuer ===========================
    if (n_steps > 0) {
      constexpr uint32_t idesc_s = umma_idesc(kBf16, 0, 0, 128, 64);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = umma_idesc(kBf16, 0, 1, 128, 64);  // P (TMEM) x V (MN-major)
      const bool leader = elect_one();
      const uint64_t desc_q = smem_desc_sw128(smem_u32(sm->q), 16, 1024);
      const uint64_t desc_k0 = smem_desc_sw128(smem_u32(sm->k[0]), 16, 1024);
      const uint64_t desc_v0 = smem_desc_sw128(smem_u32(sm->v[0]), 8192, 1024);
      bool ok = mbar_wait_warp(smem_u32(&sm->q_full), 0, abort_flag);
      int s_next = 0;  // next S tile to issue
      for (int j = 0; ok && j < n_steps; ++j) {
        const int limit = min(n_steps, j + kFwdSlots);
        while (s_next < limit) {
          const int st = s_next % kFwdStages;
          ok = mbar_wait_warp(smem_u32(&sm->kv_full[st]), (s_next / kFwdStages) & 1, abort_flag);
          if (!ok) break;
          if (leader) {
            BSA_TR(1, s_next, 0);
            const int slot = s_next % kFwdSlots;
            const uint64_t desc_k = desc_k0 + static_cast<uint64_t>(st * (kTileBytes >> 4));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ss(tmem + 64 * slot, desc_q + 2 * kk, desc_k + 2 * kk, idesc_s, kk > 0);
            tc_commit(smem_u32(&sm->s_full[slot]));
            BSA_TR(1, s_next, 1);
          }
          ++s_next;
        }
        if (!ok) break;
        const int slot = j % kFwdSlots;
        ok = mbar_wait_warp(smem_u32(&sm->p_full[slot]), (j / kFwdSlots) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          BSA_TR(1, j, 2);
          const int st = j % kFwdStages;
          const int g = j & 1;
          const uint64_t desc_v = desc_v0 + static_cast<uint64_t>(st * (kTileBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tmem + kTmemO + 64 * g, tmem + 64 * slot + 8 * kk, desc_v + 128 * kk, idesc_pv,
                    (j >= 2) || (kk > 0));
          tc_commit(smem_u32(&sm->kv_empty[st]));  // frees the stage and marks P V of step j done
          BSA_TR(1, j, 3);
        }
      }
      if (!ok) fwd_give_up(sm, p.status, kFailMma);
    }
  } else {
    // =========================== softmax + epilogue ===========================
    const int g = warp >> 2;          // softmax group: steps j = g, g+2, ...
    const int quarter = warp & 3;     // TMEM lane quarter this warp may touch
    const int half = quarter >> 1;    // which query block of the pair
    const int r_cta = quarter * 32 + lane;
    const int row = pr * 128 + r_cta;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem + lane_base + kTmemO + 64 * g;
    const float c = p.scale_log2;
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    int ent_next = g < n_steps ? __ldg(ents + g) : 0;

    for (int j = g; j < n_steps; j += 2) {
      const int ent = ent_next;
      if (j + 2 < n_steps) ent_next = __ldg(ents + j + 2);
      const int slot = j % kFwdSlots;
      const bool listed = (ent >> half) & 1;
      ok = mbar_wait_warp(smem_u32(&sm->s_full[slot]), (j / kFwdSlots) & 1, abort_flag);
      if (!ok) break;
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), j, 0);
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_base + 64 * slot;
      uint32_t pk[32];
      if (listed) {
        uint32_t sr[64];
        tmem_ld_32x32b_x32(s_addr, sr);
        tmem_ld_32x32b_x32(s_addr + 32, sr + 32);
        tc_wait_ld();
        if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), j, 1);
        float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]);
        float mx2 = __uint_as_float(sr[2]), mx3 = __uint_as_float(sr[3]);
#pragma unroll
        for (int i = 4; i < 64; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
          mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
        }
        const float zmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * c;
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
          // The group's O must hold its previous step's product (step j-2 >= 0) before it is
          // scaled.  kv_empty of that step's stage completes exactly then; its next phase belongs
          // to step j+6, which cannot complete before this warp has delivered P_j.
          ok = mbar_wait_warp(smem_u32(&sm->kv_empty[(j - 2) % kFwdStages]),
                              ((j - 2) / kFwdStages) & 1, abort_flag);
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
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
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
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = 0u;
      }
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), j, 2);
      tmem_st_32x32b_x32(s_addr, pk);  // P over the first 32 columns of the S slot
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[slot]));
      if (lane == 0 && !(warp & 1)) BSA_TR(2 + (warp >> 1), j, 3);
    }

    // ---- epilogue: merge the two groups' partial results of every row ----
    // the last P V frees the last stage; S of this warp's last step being complete implies every
    // P V more than four steps back is complete, so the awaited phase cannot be mistaken
    if (ok && n_steps > 0)
      ok = mbar_wait_warp(smem_u32(&sm->kv_empty[(n_steps - 1) % kFwdStages]),
                          ((n_steps - 1) / kFwdStages) & 1, abort_flag);
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
      // weights of accumulator 0 / 1; an accumulator that no step ever wrote is never read
      const float w0 = (g == 0 ? w_me : w_ot) * inv;
      const float w1 = (g == 0 ? w_ot : w_me) * inv;
      uint32_t packed[16];
      if (n_steps > 0) {
        tc_fence_after();
        uint32_t a0[32], a1[32];
        tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 32 * g, a0);
        if (n_steps > 1) tmem_ld_32x32b_x32(tmem + lane_base + kTmemO + 64 + 32 * g, a1);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = __uint_as_float(a0[i]) * w0, x1 = __uint_as_float(a0[i + 1]) * w0;
          if (n_steps > 1) {
            x0 = fmaf(__uint_as_float(a1[i]), w1, x0);
            x1 = fmaf(__uint_as_float(a1[i + 1]), w1, x1);
          }
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
