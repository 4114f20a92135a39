// Forward block-sparse attention for sm_100a.
//
// One CTA owns one PAIR of adjacent query blocks (128 query rows = the 128 lanes of a tcgen05
// accumulator) of one (batch, head) and walks that pair's list of key blocks:
//   warp 4 (one lane)  : TMA producer — Q once, then only the listed K/V tiles into a smem ring
//   warp 5 (one lane)  : tcgen05.mma issuer — S = Q K^T into a double-buffered TMEM tile,
//                        O += P V with P read from TMEM and V as an MN-major smem operand
//   warps 0..3         : online softmax, one thread per query row (TMEM lane): tcgen05.ld of S,
//                        exp2, P written back to TMEM as 16-bit, lazy rescale of O, epilogue
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

constexpr int kFwdStages = 5;
constexpr int kFwdThreads = 192;
constexpr uint32_t kTileBytes = 64 * 64 * 2;       // one K or V tile
constexpr uint32_t kQBytes = 128 * 64 * 2;         // one query-pair tile
constexpr uint32_t kFwdTmemCols = 256;
constexpr uint32_t kTmemS0 = 0, kTmemS1 = 64, kTmemO = 128, kTmemP0 = 192, kTmemP1 = 224;
constexpr float kRescaleThreshold = 8.0f;

struct FwdSmem {
  uint8_t q[kQBytes];
  uint8_t k[kFwdStages][kTileBytes];
  uint8_t v[kFwdStages][kTileBytes];
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_step;   // one phase per P V step
  uint64_t o_final;  // completes once, after the last P V
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
__global__ void __launch_bounds__(kFwdThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem* sm = reinterpret_cast<FwdSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = threadIdx.x >> 5;
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm->s_full[i]), 1);
      mbar_init(smem_u32(&sm->p_full[i]), 4);  // one arrival per softmax warp
    }
    mbar_init(smem_u32(&sm->o_step), 1);
    mbar_init(smem_u32(&sm->o_final), 1);
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sm->tmem_base), kFwdTmemCols);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->abort_flag;

  if (warp == 4) {
    // =========================== TMA producer ===========================
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(smem_u32(&sm->q_full), kQBytes);
      tma_load_4d(smem_u32(sm->q), &tm_q, smem_u32(&sm->q_full), 0, pr * 128, h, b);
      for (int j = 0; j < n_steps; ++j) {
        const int s = j % kFwdStages;
        const uint32_t ph = (j / kFwdStages) & 1;
        if (!mbar_wait(smem_u32(&sm->kv_empty[s]), ph ^ 1, abort_flag)) {
          fwd_give_up(sm, p.status, kFailProducer);
          break;
        }
        const int nblk = __ldg(ents + j) >> 2;
        const uint32_t bar = smem_u32(&sm->kv_full[s]);
        mbar_expect_tx(bar, 2 * kTileBytes);
        tma_load_4d(smem_u32(sm->k[s]), &tm_k, bar, 0, nblk * 64, h, b);
        tma_load_4d(smem_u32(sm->v[s]), &tm_v, bar, 0, nblk * 64, h, b);
      }
    }
  } else if (warp == 5) {
    // =========================== MMA issuer ===========================
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_s = umma_idesc(kBf16, 0, 0, 128, 64);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = umma_idesc(kBf16, 0, 1, 128, 64);  // P (TMEM) x V (MN-major)
      const uint64_t desc_q = smem_desc_sw128(smem_u32(sm->q), 16, 1024);
      bool ok = mbar_wait(smem_u32(&sm->q_full), 0, abort_flag);
      ok = ok && mbar_wait(smem_u32(&sm->kv_full[0]), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        const uint64_t desc_k = smem_desc_sw128(smem_u32(sm->k[0]), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tmem + kTmemS0, desc_q + 2 * kk, desc_k + 2 * kk, idesc_s, kk > 0);
        tc_commit(smem_u32(&sm->s_full[0]));
      }
      for (int j = 0; ok && j < n_steps; ++j) {
        const int s = j % kFwdStages;
        if (j + 1 < n_steps) {
          const int s1 = (j + 1) % kFwdStages;
          ok = mbar_wait(smem_u32(&sm->kv_full[s1]), ((j + 1) / kFwdStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t desc_k = smem_desc_sw128(smem_u32(sm->k[s1]), 16, 1024);
          const uint32_t d_s = tmem + (((j + 1) & 1) ? kTmemS1 : kTmemS0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(d_s, desc_q + 2 * kk, desc_k + 2 * kk, idesc_s, kk > 0);
          tc_commit(smem_u32(&sm->s_full[(j + 1) & 1]));
        }
        ok = mbar_wait(smem_u32(&sm->p_full[j & 1]), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t desc_v = smem_desc_sw128(smem_u32(sm->v[s]), 8192, 1024);
        const uint32_t a_p = tmem + ((j & 1) ? kTmemP1 : kTmemP0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tmem + kTmemO, a_p + 8 * kk, desc_v + 128 * kk, idesc_pv, (j > 0) || (kk > 0));
        tc_commit(smem_u32(&sm->kv_empty[s]));
        tc_commit(smem_u32(&sm->o_step));
        if (j == n_steps - 1) tc_commit(smem_u32(&sm->o_final));
      }
      if (!ok) fwd_give_up(sm, p.status, kFailMma);
    }
  } else {
    // =========================== softmax + epilogue ===========================
    const int half = warp >> 1;
    const int row = pr * 128 + warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const float c = p.scale_log2;
    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    int ent_next = n_steps > 0 ? __ldg(ents) : 0;

    for (int j = 0; j < n_steps; ++j) {
      const int ent = ent_next;
      if (j + 1 < n_steps) ent_next = __ldg(ents + j + 1);
      const int buf = j & 1;
      const bool listed = (ent >> half) & 1;
      ok = mbar_wait_warp(smem_u32(&sm->s_full[buf]), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t pk[32];
      if (listed) {
        uint32_t sr[64];
        const uint32_t s_addr = tmem + lane_base + (buf ? kTmemS1 : kTmemS0);
        tmem_ld_32x32b_x32(s_addr, sr);
        tmem_ld_32x32b_x32(s_addr + 32, sr + 32);
        tc_wait_ld();
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
          m_ref = zmax;  // first listed tile of this row: O and l are still zero
        } else if (zmax > m_ref + kRescaleThreshold) {
          alpha = ex2_approx(m_ref - zmax);
          l *= alpha;
          m_ref = zmax;
          rescale = true;
        }
        if (__any_sync(0xffffffffu, rescale)) {
          // O must hold every earlier P V product before it is scaled (j >= 1 here).
          ok = mbar_wait_warp(smem_u32(&sm->o_step), (j - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t o_addr = tmem + lane_base + kTmemO;
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
      tmem_st_32x32b_x32(tmem + lane_base + (buf ? kTmemP1 : kTmemP0), pk);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[buf]));
    }

    if (!ok) {
      fwd_give_up(sm, p.status, kFailSoftmax);
    } else {
      // ---- epilogue: O = acc / l, LSE2 = m + log2(l) ----
      uint32_t packed[32];
      if (n_steps > 0) {
        ok = mbar_wait_warp(smem_u32(&sm->o_final), 0, abort_flag);
        if (!ok) fwd_give_up(sm, p.status, kFailSoftmax);
      }
      if (ok) {
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        if (n_steps > 0) {
          tc_fence_after();
          const uint32_t o_addr = tmem + lane_base + kTmemO;
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            uint32_t orow[32];
            tmem_ld_32x32b_x32(o_addr + 32 * part, orow);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              packed[part * 16 + i / 2] = pack_2x16<kBf16>(__uint_as_float(orow[i]) * inv_l,
                                                           __uint_as_float(orow[i + 1]) * inv_l);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) packed[i] = 0u;
        }
        if (row < p.N) {
          uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.o) + b * p.o_sb +
                                                h * p.o_sh + static_cast<int64_t>(row) * p.o_sn);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2],
                                packed[4 * i + 3]);
          const int64_t ri = (static_cast<int64_t>(b) * p.H + h) * p.N + row;
          p.lse2[ri] = l > 0.f ? m_ref + lg2_approx(l) : -INFINITY;
          if (p.rowmax) p.rowmax[ri] = m_true;
        }
      }
    }
  }

  // ---- tear-down: every role arrives here, also after a give-up ----
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
}

}  // namespace bsa

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
