// Backward block-sparse attention for sm_100a: one kernel template, two instantiations.
//
//   dK/dV (kDKDV = true):  a CTA owns a PAIR of key blocks (128 keys = 128 TMEM lanes), keeps K and
//       V of the pair in shared memory and walks the pair's list of query blocks (key-pair lists):
//         S^T = K Q_m^T, dP^T = V dO_m^T            (SS MMAs, M=128, N=64)
//         P^T = exp2(S^T c - LSE2[q]), dS^T = P^T (dP^T - delta[q])   (one thread per key row)
//         dV += P^T dO_m, dK += dS^T Q_m            (TS MMAs: A from TMEM, B MN-major from smem)
//   dQ    (kDKDV = false): a CTA owns a PAIR of query blocks, keeps Q and dO of the pair resident
//       and walks the query-pair lists:
//         S = Q K_n^T, dP = dO V_n^T;  dS = exp2(S c - LSE2[row]) (dP - delta[row]);  dQ += dS K_n
//
// Formulas are those of the reference's backward (fa2_custom_mask/fa2_bwd.py:56-74, 116-130) with
// M replaced by a true base-2 log-sum-exp; the iteration space is the tile lists, not the
// reference's causal loops.  dK and dQ carry the factor sm_scale.
//
// Roles: warps 0..7 compute (lane quarter = warp % 4, column half = warp / 4), warp 8 TMA
// producer, warp 9 issues the S/dP MMAs and owns TMEM, warp 10 issues the accumulating MMAs (two
// issuers, so neither waits behind the other's barrier round trips; both run warp-wide with one
// elected lane issuing).  A block of the pair that does not list the current step's tile stores
// zeros for P/dS and skips the exponentials.
#include <math.h>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace bsa {

constexpr int kBwdStages = 4;
constexpr int kBwdThreads = 352;
constexpr uint32_t kBwdTile = 64 * 64 * 2;
constexpr uint32_t kBwdPairTile = 128 * 64 * 2;
constexpr uint32_t kBwdTmemCols = 512;
// TMEM columns: X0 = S (or S^T) x2, X1 = dP (or dP^T) x2, P x2 (16-bit), dS x2 (16-bit), two fp32
// accumulators.
constexpr uint32_t kTmX0 = 0, kTmX1 = 128, kTmP = 256, kTmDS = 320, kTmAcc0 = 384, kTmAcc1 = 448;

struct BwdSmem {
  uint8_t stat0[kBwdPairTile];
  uint8_t stat1[kBwdPairTile];
  uint8_t str0[kBwdStages][kBwdTile];
  uint8_t str1[kBwdStages][kBwdTile];
  float lse[kBwdStages][64];
  float delta[kBwdStages][64];
  uint64_t stat_full;
  uint64_t in_full[kBwdStages];
  uint64_t in_empty[kBwdStages];
  uint64_t x_full[2];
  uint64_t d_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdParams {
  const int32_t* pair_ptr;
  const int32_t* pair_ent;
  const float* lse2;
  const float* delta;
  void* out0;  // dV (dK/dV kernel only)
  void* out1;  // dK or dQ
  int64_t sb, sh, sn;
  int B, H, N, npair;
  int list_b_stride, list_h_stride;
  float scale_log2;
  float sm_scale;
  int32_t* status;
};

__device__ __forceinline__ void bwd_give_up(BwdSmem* sm, int32_t* status, int code) {
  sm->abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

template <bool kBf16>
__device__ __forceinline__ void store_half_row(void* base, int64_t elem_off, const uint32_t* acc,
                                               float scale) {
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + elem_off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
      w[t] = pack_2x16<kBf16>(__uint_as_float(acc[8 * i + 2 * t]) * scale,
                              __uint_as_float(acc[8 * i + 2 * t + 1]) * scale);
    dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <bool kBf16, bool kDKDV>
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

  const int bh = blockIdx.x / p.npair;
  // dQ: long (late) rows first; dK/dV: long (early) key columns first when the mask is causal
  const int pr = kDKDV ? (blockIdx.x % p.npair) : (p.npair - 1 - (blockIdx.x % p.npair));
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int64_t li = static_cast<int64_t>(b * p.list_b_stride + h * p.list_h_stride) * p.npair + pr;
  const int beg = __ldg(p.pair_ptr + li);
  const int n_steps = __ldg(p.pair_ptr + li + 1) - beg;
  const int32_t* ents = p.pair_ent + beg;
  const int64_t vec_base = (static_cast<int64_t>(b) * p.H + h) * p.N;  // into lse2 / delta

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm->stat_full), 1);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(smem_u32(&sm->in_full[s]), 1);
      mbar_init(smem_u32(&sm->in_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm->x_full[i]), 1);
      mbar_init(smem_u32(&sm->d_full[i]), 8);  // one arrival per compute warp
    }
    sm->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sm->tmem_base), kBwdTmemCols);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
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

  if (warp == 8) {
    // =========================== TMA producer ===========================
    if (n_steps > 0) {
      const bool leader = elect_one();
      if (leader) {
        mbar_expect_tx(smem_u32(&sm->stat_full), 2 * kBwdPairTile);
        tma_load_4d(smem_u32(sm->stat0), &tm_stat0, smem_u32(&sm->stat_full), 0, pr * 128, h, b);
        tma_load_4d(smem_u32(sm->stat1), &tm_stat1, smem_u32(&sm->stat_full), 0, pr * 128, h, b);
      }
      for (int j = 0; j < n_steps; ++j) {
        const int s = j % kBwdStages;
        const uint32_t ph = (j / kBwdStages) & 1;
        const int blk = __ldg(ents + j) >> 2;
        if (!mbar_wait_warp(smem_u32(&sm->in_empty[s]), ph ^ 1, abort_flag)) {
          bwd_give_up(sm, p.status, 1);
          break;
        }
        if (leader) {
          const uint32_t bar = smem_u32(&sm->in_full[s]);
          mbar_expect_tx(bar, 2 * kBwdTile + (kDKDV ? 512u : 0u));
          tma_load_4d(smem_u32(sm->str0[s]), &tm_str0, bar, 0, blk * 64, h, b);
          tma_load_4d(smem_u32(sm->str1[s]), &tm_str1, bar, 0, blk * 64, h, b);
          if constexpr (kDKDV) {
            bulk_load_1d(smem_u32(sm->lse[s]), p.lse2 + vec_base + blk * 64, 256, bar);
            bulk_load_1d(smem_u32(sm->delta[s]), p.delta + vec_base + blk * 64, 256, bar);
          }
        }
      }
    }
  } else if (warp == 9) {
    // =========================== S / dP issuer ===========================
    if (n_steps > 0) {
      constexpr uint32_t idesc_x = umma_idesc(kBf16, 0, 0, 128, 64);
      const bool leader = elect_one();
      const uint64_t desc_a0 = smem_desc_sw128(smem_u32(sm->stat0), 16, 1024);
      const uint64_t desc_a1 = smem_desc_sw128(smem_u32(sm->stat1), 16, 1024);
      const uint64_t desc_b0 = smem_desc_sw128(smem_u32(sm->str0[0]), 16, 1024);
      const uint64_t desc_b1 = smem_desc_sw128(smem_u32(sm->str1[0]), 16, 1024);
      bool ok = mbar_wait_warp(smem_u32(&sm->stat_full), 0, abort_flag);
      for (int j = 0; ok && j < n_steps; ++j) {
        const int s = j % kBwdStages;
        const int buf = j & 1;
        ok = mbar_wait_warp(smem_u32(&sm->in_full[s]), (j / kBwdStages) & 1, abort_flag);
        if (!ok) break;
        if (j >= 2) {
          // buffer `buf` still feeds the accumulating MMAs of step j-2 (P, dS live there too)
          const int jp = j - 2;
          ok = mbar_wait_warp(smem_u32(&sm->in_empty[jp % kBwdStages]), (jp / kBwdStages) & 1,
                              abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        if (leader) {
          const uint64_t b0 = desc_b0 + static_cast<uint64_t>(s * (kBwdTile >> 4));
          const uint64_t b1 = desc_b1 + static_cast<uint64_t>(s * (kBwdTile >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + kTmX0 + 64 * buf, desc_a0 + 2 * kk, b0 + 2 * kk, idesc_x, kk > 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem + kTmX1 + 64 * buf, desc_a1 + 2 * kk, b1 + 2 * kk, idesc_x, kk > 0);
          tc_commit(smem_u32(&sm->x_full[buf]));
        }
      }
      if (!ok) bwd_give_up(sm, p.status, 2);
    }
  } else if (warp == 10) {
    // =========================== accumulating-MMA issuer ===========================
    if (n_steps > 0) {
      constexpr uint32_t idesc_acc = umma_idesc(kBf16, 0, 1, 128, 64);
      const bool leader = elect_one();
      const uint64_t desc_m0 = smem_desc_sw128(smem_u32(sm->str0[0]), 8192, 1024);
      const uint64_t desc_m1 = smem_desc_sw128(smem_u32(sm->str1[0]), 8192, 1024);
      bool ok = true;
      for (int j = 0; ok && j < n_steps; ++j) {
        const int s = j % kBwdStages;
        const int buf = j & 1;
        ok = mbar_wait_warp(smem_u32(&sm->d_full[buf]), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          const uint32_t acc_on = (j > 0) ? 1u : 0u;
          if constexpr (kDKDV) {
            const uint64_t bmn = desc_m1 + static_cast<uint64_t>(s * (kBwdTile >> 4));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ts(tmem + kTmAcc0, tmem + kTmP + 32 * buf + 8 * kk, bmn + 128 * kk, idesc_acc,
                      acc_on | (kk > 0));
          }
          const uint64_t bmn = desc_m0 + static_cast<uint64_t>(s * (kBwdTile >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tmem + kTmAcc1, tmem + kTmDS + 32 * buf + 8 * kk, bmn + 128 * kk, idesc_acc,
                    acc_on | (kk > 0));
          tc_commit(smem_u32(&sm->in_empty[s]));  // stage free; X/P/dS buffer free; acc updated
        }
      }
      if (!ok) bwd_give_up(sm, p.status, 2);
    }
  } else {
    // =========================== compute warps ===========================
    const int quarter = warp & 3;
    const int ch = warp >> 2;           // which 32 of the 64 tile columns
    const int half = quarter >> 1;      // which block of the pair this row belongs to
    const int row = pr * 128 + quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float c = p.scale_log2;
    float my_lse = 0.f, my_delta = 0.f;
    if constexpr (!kDKDV) {
      if (row < p.N) {
        my_lse = __ldg(p.lse2 + vec_base + row);
        my_delta = __ldg(p.delta + vec_base + row);
      }
    }
    bool ok = true;
    int ent_next = n_steps > 0 ? __ldg(ents) : 0;
    for (int j = 0; j < n_steps; ++j) {
      const int ent = ent_next;
      if (j + 1 < n_steps) ent_next = __ldg(ents + j + 1);
      const int s = j % kBwdStages;
      const int buf = j & 1;
      const bool listed = (ent >> half) & 1;
      if constexpr (kDKDV) {
        // the LSE2/delta vectors of this stage arrive through the async proxy
        ok = mbar_wait_warp(smem_u32(&sm->in_full[s]), (j / kBwdStages) & 1, abort_flag);
        if (!ok) break;
      }
      ok = mbar_wait_warp(smem_u32(&sm->x_full[buf]), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t pk_p[16], pk_ds[16];
      if (listed) {
        uint32_t xs[32], xd[32];
        tmem_ld_32x32b_x32(tmem + lane_base + kTmX0 + 64 * buf + 32 * ch, xs);
        tmem_ld_32x32b_x32(tmem + lane_base + kTmX1 + 64 * buf + 32 * ch, xd);
        tc_wait_ld();
        const float4* lse4 = reinterpret_cast<const float4*>(&sm->lse[s][32 * ch]);
        const float4* del4 = reinterpret_cast<const float4*>(&sm->delta[s][32 * ch]);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float l[4], d[4];
          if constexpr (kDKDV) {
            const float4 lv = lse4[i / 4], dv = del4[i / 4];
            l[0] = lv.x; l[1] = lv.y; l[2] = lv.z; l[3] = lv.w;
            d[0] = dv.x; d[1] = dv.y; d[2] = dv.z; d[3] = dv.w;
          } else {
            l[0] = l[1] = l[2] = l[3] = my_lse;
            d[0] = d[1] = d[2] = d[3] = my_delta;
          }
          float pv[4], dsv[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            pv[t] = ex2_approx(fmaf(__uint_as_float(xs[i + t]), c, -l[t]));
            dsv[t] = pv[t] * (__uint_as_float(xd[i + t]) - d[t]);
          }
          pk_p[i / 2] = pack_2x16<kBf16>(pv[0], pv[1]);
          pk_p[i / 2 + 1] = pack_2x16<kBf16>(pv[2], pv[3]);
          pk_ds[i / 2] = pack_2x16<kBf16>(dsv[0], dsv[1]);
          pk_ds[i / 2 + 1] = pack_2x16<kBf16>(dsv[2], dsv[3]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk_p[i] = 0u;
          pk_ds[i] = 0u;
        }
      }
      if constexpr (kDKDV) tmem_st_32x32b_x16(tmem + lane_base + kTmP + 32 * buf + 16 * ch, pk_p);
      tmem_st_32x32b_x16(tmem + lane_base + kTmDS + 32 * buf + 16 * ch, pk_ds);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->d_full[buf]));
    }

    if (!ok) {
      bwd_give_up(sm, p.status, 3);
    } else {
      if (n_steps > 0) {
        ok = mbar_wait_warp(smem_u32(&sm->in_empty[(n_steps - 1) % kBwdStages]),
                            ((n_steps - 1) / kBwdStages) & 1, abort_flag);
        if (!ok) bwd_give_up(sm, p.status, 3);
      }
      if (ok) {
        uint32_t acc[32];
        const int64_t off = b * p.sb + h * p.sh + static_cast<int64_t>(row) * p.sn + 32 * ch;
        if constexpr (kDKDV) {
          if (n_steps > 0) {
            tc_fence_after();
            tmem_ld_32x32b_x32(tmem + lane_base + kTmAcc0 + 32 * ch, acc);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0u;
          }
          if (row < p.N) store_half_row<kBf16>(p.out0, off, acc, 1.0f);
        }
        if (n_steps > 0) {
          tc_fence_after();
          tmem_ld_32x32b_x32(tmem + lane_base + kTmAcc1 + 32 * ch, acc);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = 0u;
        }
        if (row < p.N) store_half_row<kBf16>(p.out1, off, acc, p.sm_scale);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

template <bool kDKDV>
static int launch_bwd(const void* q, const void* k, const void* v, const void* dout,
                      const int64_t strides[4], const float* lse2, const float* delta, void* out0,
                      void* out1, const int32_t* pair_ptr, const int32_t* pair_ent,
                      int list_b_stride, int list_h_stride, float sm_scale, int dtype, int B, int H,
                      int N, int D, int32_t* status, void* stream) {
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!lse2 || !delta || !pair_ptr || !pair_ent || !is_aligned(lse2, 16) || !is_aligned(delta, 16))
    return BSA_ERR_BAD_POINTER;
  int rc;
  const void* ops[6] = {q, k, v, dout, out1, kDKDV ? out0 : out1};
  for (const void* op : ops)
    if ((rc = check_qkv_operand(op, strides)) != BSA_OK) return rc;
  if ((rc = check_device_sm100()) != BSA_OK) return rc;
  const int nb = N / kBlock;
  const int npair = (nb + 1) / 2;
  if (static_cast<int64_t>(B) * H * npair > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  // dK/dV: K, V resident; Q, dO streamed.   dQ: Q, dO resident; K, V streamed.
  const void* stat0 = kDKDV ? k : q;
  const void* stat1 = kDKDV ? v : dout;
  const void* str0 = kDKDV ? q : k;
  const void* str1 = kDKDV ? dout : v;
  CUtensorMap tm_a0, tm_a1, tm_b0, tm_b1;
  if ((rc = make_qkv_tmap(&tm_a0, stat0, strides, B, H, N, dtype, 128)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_a1, stat1, strides, B, H, N, dtype, 128)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_b0, str0, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;
  if ((rc = make_qkv_tmap(&tm_b1, str1, strides, B, H, N, dtype, 64)) != BSA_OK) return rc;

  BwdParams prm;
  prm.pair_ptr = pair_ptr;
  prm.pair_ent = pair_ent;
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
  prm.npair = npair;
  prm.list_b_stride = list_b_stride;
  prm.list_h_stride = list_h_stride;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.sm_scale = sm_scale;
  prm.status = status;

  const size_t smem_bytes = sizeof(BwdSmem) + 1024;
  auto kern = dtype == BSA_BF16 ? attn_bwd_kernel<true, kDKDV> : attn_bwd_kernel<false, kDKDV>;
  if ((rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes)) != BSA_OK)
    return rc;
  const dim3 grid(static_cast<unsigned>(B * H * npair));
  kern<<<grid, kBwdThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tm_a0, tm_a1, tm_b0,
                                                                             tm_b1, prm);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}

}  // namespace bsa

extern "C" int bsa_attn_bwd_dkdv(const void* q, const void* k, const void* v, const void* dout,
                                 const int64_t strides[4], const float* lse2, const float* delta,
                                 void* dk, void* dv, const int32_t* kpair_ptr,
                                 const int32_t* kpair_ent, int list_b_stride, int list_h_stride,
                                 float sm_scale, int dtype, int B, int H, int N, int D,
                                 int32_t* status, void* stream) {
  return bsa::launch_bwd<true>(q, k, v, dout, strides, lse2, delta, dv, dk, kpair_ptr, kpair_ent,
                               list_b_stride, list_h_stride, sm_scale, dtype, B, H, N, D, status,
                               stream);
}

extern "C" int bsa_attn_bwd_dq(const void* q, const void* k, const void* v, const void* dout,
                               const int64_t strides[4], const float* lse2, const float* delta,
                               void* dq, const int32_t* qpair_ptr, const int32_t* qpair_ent,
                               int list_b_stride, int list_h_stride, float sm_scale, int dtype,
                               int B, int H, int N, int D, int32_t* status, void* stream) {
  return bsa::launch_bwd<false>(q, k, v, dout, strides, lse2, delta, nullptr, dq, qpair_ptr,
                                qpair_ent, list_b_stride, list_h_stride, sm_scale, dtype, B, H, N,
                                D, status, stream);
}
