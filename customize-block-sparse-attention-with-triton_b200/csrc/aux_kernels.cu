// HBM-bound helpers around the attention kernels:
//   bsa_attn_bwd_delta   delta = rowsum(O * dO) in fp32
//   bsa_reorder / bsa_inv_reorder   head-wise permutation of the (F, H, W) token grid
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace bsa {

// ---------------------------------------------------------------------------------------------
// delta
// ---------------------------------------------------------------------------------------------
// Eight lanes own one 128-byte row (64 16-bit values): a warp covers 4 rows per step and a CTA of
// 8 warps covers 128 rows with 4 independent steps in flight per thread.
constexpr int kDeltaThreads = 256;
constexpr int kDeltaRowsPerCta = 128;

template <bool kBf16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa, fb;
    if constexpr (kBf16) {
      fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
      fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
    } else {
      fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
      fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
    }
    acc = fmaf(fa.x, fb.x, acc);
    acc = fmaf(fa.y, fb.y, acc);
  }
  return acc;
}

template <bool kBf16>
__global__ void __launch_bounds__(kDeltaThreads)
bwd_delta_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dout, int64_t sb,
                 int64_t sh, int64_t sn, float* __restrict__ delta, int H, int N, int64_t rows) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane >> 3, chunk = lane & 7;
  // A warp's 16 rows lie in one (batch, head): N is a multiple of 64 and the warp starts at a
  // multiple of 16, so the division is done once per thread, not once per row.
  const int64_t warp_row = static_cast<int64_t>(blockIdx.x) * kDeltaRowsPerCta + warp * 16;
  const int64_t row0 = warp_row + sub;
  const int64_t bh = warp_row / N;
  const int64_t n0 = warp_row - bh * N + sub;
  const int64_t b = bh / H;
  const int64_t base = b * sb + (bh - b * H) * sh + chunk * 8;
  uint4 xo[4], xd[4];
  bool live[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    live[i] = row0 + 4 * i < rows;
    if (live[i]) {
      const int64_t off = base + (n0 + 4 * i) * sn;
      xo[i] = __ldg(reinterpret_cast<const uint4*>(o + off));
      xd[i] = __ldg(reinterpret_cast<const uint4*>(dout + off));
    } else {
      xo[i] = make_uint4(0, 0, 0, 0);
      xd[i] = make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float acc = dot8<kBf16>(xo[i], xd[i]);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (chunk == 0 && live[i]) delta[row0 + 4 * i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// head-wise token reorder
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int pick3(int sel, int v0, int v1, int v2) {
  return sel == 0 ? v0 : (sel == 1 ? v1 : (sel == 2 ? v2 : 0));
}

// Destination token of source token t for head order (p0,p1,p2) over a grid of extents
// (e0,e1,e2): the coordinates are re-laid-out in the order (p0,p1,p2).
__device__ __forceinline__ int permuted_token(int t, int e0, int e1, int e2, int p0, int p1,
                                              int p2) {
  const int plane = e1 * e2;
  const int c_f = t / plane;
  const int rem = t - c_f * plane;
  const int c_h = rem / e2;
  const int c_w = rem - c_h * e2;
  const int c0 = pick3(p0, c_f, c_h, c_w);
  const int c1 = pick3(p1, c_f, c_h, c_w);
  const int c2 = pick3(p2, c_f, c_h, c_w);
  const int d1 = pick3(p1, e0, e1, e2);
  const int d2 = pick3(p2, e0, e1, e2);
  return c0 * (d1 * d2) + c1 * d2 + c2;
}

constexpr int kReorderThreads = 256;
constexpr int kReorderPieces = 4;  // independent loads in flight per thread

// A CTA moves kReorderThreads * kReorderPieces Vec-sized pieces of the token rows of one
// (batch, head) (blockIdx.y, strided if the grid's y extent is smaller than batch * heads): all
// index arithmetic is 32-bit and the head's axis order is read once per CTA.  Every thread issues
// its loads before its stores.  kInverse: the source grid has the extents permuted by `orders`,
// and `inv_orders` lays the coordinates back out.
template <typename Vec, bool kInverse>
__global__ void __launch_bounds__(kReorderThreads)
reorder_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t sb, int64_t sh,
               int64_t st, int64_t ob, int64_t oh, int64_t ot, const int32_t* __restrict__ orders,
               const int32_t* __restrict__ inv_orders, int heads, int n_bh, int T, int F, int Hh,
               int W, int vec_per_row) {
  const uint32_t per_head = static_cast<uint32_t>(T) * static_cast<uint32_t>(vec_per_row);
  const uint32_t first = blockIdx.x * (kReorderThreads * kReorderPieces) + threadIdx.x;
  for (int bh = blockIdx.y; bh < n_bh; bh += gridDim.y) {
    const int h = bh % heads;
    const int b = bh / heads;
    const int o0 = __ldg(orders + 3 * h), o1 = __ldg(orders + 3 * h + 1),
              o2 = __ldg(orders + 3 * h + 2);
    int e0 = F, e1 = Hh, e2 = W, p0 = o0, p1 = o1, p2 = o2;
    if constexpr (kInverse) {
      e0 = pick3(o0, F, Hh, W);
      e1 = pick3(o1, F, Hh, W);
      e2 = pick3(o2, F, Hh, W);
      p0 = __ldg(inv_orders + 3 * h);
      p1 = __ldg(inv_orders + 3 * h + 1);
      p2 = __ldg(inv_orders + 3 * h + 2);
    }
    // An order row that is not a permutation of (0, 1, 2) would send tokens past the end of the
    // head (the reference has no check either): such a head's rows are left unwritten.
    const bool valid = ((1 << p0) | (1 << p1) | (1 << p2)) == 7 && (p0 | p1 | p2) >= 0 &&
                       (!kInverse || (((1 << o0) | (1 << o1) | (1 << o2)) == 7 && (o0 | o1 | o2) >= 0));
    if (!valid) continue;
    const uint8_t* src = in + b * sb + h * sh;  // byte offsets
    uint8_t* dst = out + b * ob + h * oh;
    Vec val[kReorderPieces];
    int64_t to[kReorderPieces];
#pragma unroll
    for (int i = 0; i < kReorderPieces; ++i) {
      const uint32_t idx = first + i * kReorderThreads;
      to[i] = -1;
      if (idx < per_head) {
        const int t = static_cast<int>(idx / static_cast<uint32_t>(vec_per_row));
        const int piece = static_cast<int>(idx - static_cast<uint32_t>(t) * vec_per_row);
        val[i] = *reinterpret_cast<const Vec*>(src + t * st + piece * sizeof(Vec));
        to[i] = permuted_token(t, e0, e1, e2, p0, p1, p2) * ot + piece * sizeof(Vec);
      }
    }
#pragma unroll
    for (int i = 0; i < kReorderPieces; ++i)
      if (to[i] >= 0) *reinterpret_cast<Vec*>(dst + to[i]) = val[i];
  }
}

template <bool kInverse>
static int launch_reorder(const void* in, const int64_t s[4], void* out, const int64_t so[4],
                          const int32_t* orders, const int32_t* inv_orders, int B, int heads, int T, int D, int F, int Hh,
                          int W, int elem_bytes, void* stream) {
  if (B <= 0 || heads <= 0 || T <= 0 || D <= 0 || F <= 0 || Hh <= 0 || W <= 0 ||
      static_cast<int64_t>(F) * Hh * W != T)
    return BSA_ERR_BAD_SHAPE;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
    return BSA_ERR_BAD_DTYPE;
  if (!in || !out || !orders || (kInverse && !inv_orders)) return BSA_ERR_BAD_POINTER;
  if (!s || !so) return BSA_ERR_BAD_POINTER;
  if (s[3] != 1 || s[0] < 0 || s[1] < 0 || s[2] < 0) return BSA_ERR_BAD_STRIDE;
  if (so[3] != 1 || so[0] < 0 || so[1] < 0 || so[2] < 0) return BSA_ERR_BAD_STRIDE;
  const int64_t row_bytes = static_cast<int64_t>(D) * elem_bytes;
  const int64_t sb = s[0] * elem_bytes, sh = s[1] * elem_bytes, st = s[2] * elem_bytes;
  const int64_t ob = so[0] * elem_bytes, oh = so[1] * elem_bytes, ot = so[2] * elem_bytes;
  // widest piece that divides the row and keeps every access aligned
  int vec = 16;
  auto fits = [&](int v) {
    return row_bytes % v == 0 && sb % v == 0 && sh % v == 0 && st % v == 0 && ob % v == 0 &&
           oh % v == 0 && ot % v == 0 && is_aligned(in, v) && is_aligned(out, v);
  };
  while (vec > elem_bytes && !fits(vec)) vec >>= 1;
  if (!fits(vec)) return BSA_ERR_BAD_POINTER;
  const int vec_per_row = static_cast<int>(row_bytes / vec);
  const int64_t per_head = static_cast<int64_t>(T) * vec_per_row;
  const int64_t n_bh = static_cast<int64_t>(B) * heads;
  if (per_head > 0x7fffffffLL || n_bh > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;
  constexpr int kPerCta = kReorderThreads * kReorderPieces;
  const dim3 g(static_cast<unsigned>((per_head + kPerCta - 1) / kPerCta),
               static_cast<unsigned>(n_bh < 65535 ? n_bh : 65535));
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const uint8_t* pi = static_cast<const uint8_t*>(in);
  uint8_t* po = static_cast<uint8_t*>(out);
#define BSA_LAUNCH_REORDER(V)                                                                      \
  reorder_kernel<V, kInverse><<<g, kReorderThreads, 0, cs>>>(pi, po, sb, sh, st, ob, oh, ot,       \
                                                             orders, inv_orders, heads,            \
                                                             static_cast<int>(n_bh), T, F, Hh, W,  \
                                                             vec_per_row)
  switch (vec) {
    case 16: BSA_LAUNCH_REORDER(uint4); break;
    case 8: BSA_LAUNCH_REORDER(uint2); break;
    case 4: BSA_LAUNCH_REORDER(uint32_t); break;
    case 2: BSA_LAUNCH_REORDER(uint16_t); break;
    default: BSA_LAUNCH_REORDER(uint8_t); break;
  }
#undef BSA_LAUNCH_REORDER
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}

}  // namespace bsa

extern "C" int bsa_attn_bwd_delta(const void* o, const void* dout, const int64_t s[4], float* delta,
                                  int dtype, int B, int H, int N, int D, void* stream) {
  using namespace bsa;
  if (B <= 0 || H <= 0 || N <= 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if (dtype != BSA_F16 && dtype != BSA_BF16) return BSA_ERR_BAD_DTYPE;
  if (!delta) return BSA_ERR_BAD_POINTER;
  int rc;
  if ((rc = check_qkv_operand(o, s)) != BSA_OK) return rc;
  if ((rc = check_qkv_operand(dout, s)) != BSA_OK) return rc;
  const int64_t rows = static_cast<int64_t>(B) * H * N;
  const int64_t blocks = (rows + kDeltaRowsPerCta - 1) / kDeltaRowsPerCta;
  if (blocks > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const uint16_t* po = static_cast<const uint16_t*>(o);
  const uint16_t* pd = static_cast<const uint16_t*>(dout);
  if (dtype == BSA_BF16)
    bwd_delta_kernel<true><<<static_cast<unsigned>(blocks), kDeltaThreads, 0, cs>>>(
        po, pd, s[0], s[1], s[2], delta, H, N, rows);
  else
    bwd_delta_kernel<false><<<static_cast<unsigned>(blocks), kDeltaThreads, 0, cs>>>(
        po, pd, s[0], s[1], s[2], delta, H, N, rows);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}

extern "C" int bsa_reorder(const void* in, void* out, const int64_t strides[4],
                           const int32_t* orders, int B, int heads, int T, int D, int F, int Hh,
                           int W, int elem_bytes, void* stream) {
  return bsa::launch_reorder<false>(in, strides, out, strides, orders, nullptr, B, heads, T, D, F,
                                    Hh, W, elem_bytes, stream);
}

extern "C" int bsa_reorder_strided(const void* in, const int64_t in_strides[4], void* out,
                                   const int64_t out_strides[4], const int32_t* orders, int B,
                                   int heads, int T, int D, int F, int Hh, int W, int elem_bytes,
                                   void* stream) {
  return bsa::launch_reorder<false>(in, in_strides, out, out_strides, orders, nullptr, B, heads, T,
                                    D, F, Hh, W, elem_bytes, stream);
}

extern "C" int bsa_inv_reorder(const void* in, void* out, const int64_t strides[4],
                               const int32_t* orders, const int32_t* inv_orders, int B, int heads,
                               int T, int D, int F, int Hh, int W, int elem_bytes, void* stream) {
  return bsa::launch_reorder<true>(in, strides, out, strides, orders, inv_orders, B, heads, T, D, F,
                                   Hh, W, elem_bytes, stream);
}

extern "C" int bsa_inv_reorder_strided(const void* in, const int64_t in_strides[4], void* out,
                                       const int64_t out_strides[4], const int32_t* orders,
                                       const int32_t* inv_orders, int B, int heads, int T, int D,
                                       int F, int Hh, int W, int elem_bytes, void* stream) {
  return bsa::launch_reorder<true>(in, in_strides, out, out_strides, orders, inv_orders, B, heads,
                                   T, D, F, Hh, W, elem_bytes, stream);
}
