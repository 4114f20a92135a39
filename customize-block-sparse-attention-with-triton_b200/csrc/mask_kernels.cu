// Mask preprocessing on the device (HBM-bound byte/integer work):
//   bsa_mask_reduce      dense [.., N, N] boolean mask  ->  [.., nb, nb] block mask (any over 64x64)
//   bsa_tile_lists_build block mask -> CSR, transposed CSR and the reference's (groups, n_list)
//                        layout, with three launches (one, for the row lists of a small mask
//                        alone) and no host synchronisation.
#include "host_common.h"

namespace bsa {

// ---------------------------------------------------------------------------------------------
// dense -> block
// ---------------------------------------------------------------------------------------------
// CTA tile: 64 rows x 1024 columns (16 blocks).  Thread t streams the 16-byte column segment
// (t & 63) of rows (t >> 6) + 4 i, i = 0..15: 16 independent 128-bit loads in flight per thread.
constexpr int kReduceThreads = 256;
constexpr int kReduceCols = 1024;

__device__ __forceinline__ uint4 ld_stream_u4(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint32_t zero_byte_bits(uint32_t x) {
  return (x - 0x01010101u) & ~x & 0x80808080u;  // non-zero iff some byte of x is zero
}

__global__ void __launch_bounds__(kReduceThreads)
mask_reduce_kernel(const uint8_t* __restrict__ dense, int64_t sb, int64_t sh, int64_t sr, int H,
                   int N, int nb, uint8_t* __restrict__ block, int32_t* partial, int mark_partial) {
  __shared__ uint32_t s_any[4][16];
  __shared__ uint32_t s_zero[4][16];
  const int bh = blockIdx.z;
  const int b = bh / H, h = bh % H;
  const int rb = blockIdx.y;
  const int col0 = blockIdx.x * kReduceCols;
  const int seg = threadIdx.x & 63;
  const int rg = threadIdx.x >> 6;
  const int col = col0 + seg * 16;
  uint32_t any_bits = 0, zero_bits = 0;
  if (col < N) {
    const uint8_t* base = dense + b * sb + h * sh + static_cast<int64_t>(rb) * 64 * sr + col;
    uint4 x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = ld_stream_u4(base + static_cast<int64_t>(rg + 4 * i) * sr);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      any_bits |= x[i].x | x[i].y | x[i].z | x[i].w;
      zero_bits |= zero_byte_bits(x[i].x) | zero_byte_bits(x[i].y) | zero_byte_bits(x[i].z) |
                   zero_byte_bits(x[i].w);
    }
  }
  // four neighbouring lanes hold the four 16-byte quarters of one block's 64 columns
  any_bits |= __shfl_xor_sync(0xffffffffu, any_bits, 1);
  any_bits |= __shfl_xor_sync(0xffffffffu, any_bits, 2);
  zero_bits |= __shfl_xor_sync(0xffffffffu, zero_bits, 1);
  zero_bits |= __shfl_xor_sync(0xffffffffu, zero_bits, 2);
  if ((seg & 3) == 0) {
    s_any[rg][seg >> 2] = any_bits;
    s_zero[rg][seg >> 2] = zero_bits;
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int t = threadIdx.x;
    const int cb = col0 / 64 + t;
    const bool any = (s_any[0][t] | s_any[1][t] | s_any[2][t] | s_any[3][t]) != 0;
    const bool has_zero = (s_zero[0][t] | s_zero[1][t] | s_zero[2][t] | s_zero[3][t]) != 0;
    const bool in_range = cb < nb;
    // 0 = no element kept, 1 = kept; with mark_partial a kept tile that also has masked elements is 2
    if (in_range)
      block[(static_cast<int64_t>(bh) * nb + rb) * nb + cb] =
          any ? ((mark_partial && has_zero) ? 2 : 1) : 0;
    if (partial) {
      const unsigned m = __ballot_sync(0x0000ffffu, in_range && any && has_zero);
      if (t == 0 && m) atomicAdd(partial, __popc(m));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// block mask -> tile lists
// ---------------------------------------------------------------------------------------------
// Two list kinds share one code path.  "major" is the axis a list belongs to, "minor" the axis
// it enumerates (ascending).
//   kind 0 rows   : major = query block,      minor = key block     -> row_ptr / col_idx
//   kind 1 cols   : major = key block,        minor = query block   -> col_ptr / row_idx
// Pass 1 writes per-major counts into ptr[], the scan turns them into offsets in place (ptr[n] =
// total), pass 2 writes the entries.
struct ListArgs {
  const uint8_t* block;
  int64_t s0, s1, s2, s3;
  int B, H, nb;
  int32_t* ptr[2];
  int32_t* ent[2];
  int32_t* groups;
  int32_t* meta;
};

constexpr int kListThreads = 256;

// Mask byte of tile (row, col): 0 = not kept, 1 = kept, 2 = kept with masked elements inside (a
// dense mask reduced with mark_partial).  A list entry of such a tile carries kPartialFlag.
__device__ __forceinline__ int list_byte(const ListArgs& a, const uint8_t* head, int row, int col) {
  return head[row * a.s2 + col * a.s3];
}
__device__ __forceinline__ int list_entry(int index, int byte) {
  return byte == 2 ? (index | BSA_LIST_PARTIAL_FLAG) : index;
}

// Lists along the mask's rows: one warp per major unit, lanes sweep the minor axis 32 at a time.
template <bool kFill>
__device__ __forceinline__ void lists_along_rows(const ListArgs& a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * (kListThreads / 32) + warp;
  if (unit >= static_cast<int64_t>(a.B) * a.H * a.nb) return;
  const int bh = static_cast<int>(unit / a.nb);
  const int major = static_cast<int>(unit % a.nb);
  const uint8_t* head = a.block + (bh / a.H) * a.s0 + (bh % a.H) * a.s1;
  int count = 0;
  int32_t* out = nullptr;
  if constexpr (kFill) out = a.ent[0] + a.ptr[0][unit];
  // 128 columns per pass, four independent loads per lane, the next pass's loads asked for before
  // this pass's ballots: a row costs about one round trip to memory, not one per 32 columns
  int byte[4], next[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = 32 * j + lane;
    next[j] = c < a.nb ? list_byte(a, head, major, c) : 0;
  }
  for (int c0 = 0; c0 < a.nb; c0 += 128) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      byte[j] = next[j];
      const int c = c0 + 128 + 32 * j + lane;
      next[j] = c < a.nb ? list_byte(a, head, major, c) : 0;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool f = byte[j] != 0;
      const unsigned m = __ballot_sync(0xffffffffu, f);
      if constexpr (kFill) {
        if (f)
          out[count + __popc(m & ((1u << lane) - 1u))] = list_entry(c0 + 32 * j + lane, byte[j]);
      }
      count += __popc(m);
    }
  }
  if constexpr (!kFill) {
    if (lane == 0) a.ptr[0][unit] = count;
  }
}

// Lists along the mask's columns: one CTA per 32 major units (lane = unit, so a warp reads
// consecutive bytes of a mask row); the 8 warps split the minor axis into contiguous chunks.
template <bool kFill>
__device__ __forceinline__ void lists_along_cols(const ListArgs& a) {
  __shared__ int s_cnt[kListThreads / 32][33];
  const int groups_per_head = (a.nb + 31) / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t g = blockIdx.x;
  if (g >= static_cast<int64_t>(a.B) * a.H * groups_per_head) return;  // whole CTA leaves
  const int bh = static_cast<int>(g / groups_per_head);
  const int major = static_cast<int>(g % groups_per_head) * 32 + lane;
  const bool valid = major < a.nb;
  const uint8_t* head = a.block + (bh / a.H) * a.s0 + (bh % a.H) * a.s1;
  constexpr int kWarps = kListThreads / 32;
  const int chunk = (a.nb + kWarps - 1) / kWarps;
  const int r0 = warp * chunk;
  const int r1 = min(a.nb, r0 + chunk);
  // eight rows per batch: eight independent loads in flight per thread instead of one
  int count = 0;
  if (valid) {
    int r = r0;
    for (; r + 8 <= r1; r += 8) {
      int b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = list_byte(a, head, r + j, major);
#pragma unroll
      for (int j = 0; j < 8; ++j) count += b[j] != 0 ? 1 : 0;
    }
    for (; r < r1; ++r) count += list_byte(a, head, r, major) != 0 ? 1 : 0;
  }
  s_cnt[warp][lane] = count;
  __syncthreads();
  const int64_t unit = static_cast<int64_t>(bh) * a.nb + major;
  if constexpr (!kFill) {
    if (warp == 0 && valid) {
      int total = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) total += s_cnt[w][lane];
      a.ptr[1][unit] = total;
    }
  } else {
    if (valid) {
      int before = 0;
      for (int w = 0; w < warp; ++w) before += s_cnt[w][lane];
      int32_t* out = a.ent[1] + a.ptr[1][unit] + before;
      int k = 0;
      int r = r0;
      for (; r + 8 <= r1; r += 8) {
        int b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = list_byte(a, head, r + j, major);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (b[j] != 0) out[k++] = list_entry(r + j, b[j]);
      }
      for (; r < r1; ++r) {
        const int byte = list_byte(a, head, r, major);
        if (byte != 0) out[k++] = list_entry(r, byte);
      }
    }
  }
}

template <bool kFill>
__global__ void __launch_bounds__(kListThreads) lists_pass_kernel(const ListArgs a) {
  const int kind = blockIdx.y;
  if (a.ptr[kind] == nullptr) return;
  if (kind == 0) lists_along_rows<kFill>(a);
  else lists_along_cols<kFill>(a);
}

// In-place exclusive scan of the counts of one list kind per CTA; kind 0 also emits the
// reference's `groups` rows (b, h, m, start, len) for the non-empty rows, in row order.
constexpr int kScanThreads = 1024;

__device__ __forceinline__ int block_exclusive_scan(int v, int* s_warp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  __syncthreads();  // protects s_warp between consecutive calls
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = s_warp[lane];
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += t;
    }
    s_warp[lane] = wi - w;
    if (lane == 31) s_warp[32] = wi;
  }
  __syncthreads();
  *total = s_warp[32];
  return s_warp[warp] + incl - v;
}

__global__ void __launch_bounds__(kScanThreads) lists_scan_kernel(const ListArgs a) {
  __shared__ int s_warp[33];
  const int kind = blockIdx.x;
  int32_t* ptr = a.ptr[kind];
  if (ptr == nullptr) return;  // meta was cleared by the host side
  const int64_t n = static_cast<int64_t>(a.B) * a.H * a.nb;
  const bool want_groups = (kind == 0 && a.groups != nullptr);
  // Tiles of 8 counts per thread, held in registers between the two block scans and the
  // write-back, so every count is read once and no load waits for another.
  constexpr int kPer = 8;
  int carry = 0, gcarry = 0;
  for (int64_t base = 0; base < n; base += static_cast<int64_t>(kScanThreads) * kPer) {
    const int64_t i0 = base + static_cast<int64_t>(threadIdx.x) * kPer;
    int c[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) c[j] = i0 + j < n ? ptr[i0 + j] : 0;
    int sum = 0, nonempty = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      sum += c[j];
      nonempty += c[j] > 0;
    }
    int total = 0, gtotal = 0;
    int run = carry + block_exclusive_scan(sum, s_warp, &total);
    int grun = 0;
    if (kind == 0) grun = gcarry + block_exclusive_scan(nonempty, s_warp, &gtotal);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int64_t i = i0 + j;
      if (i < n) {
        ptr[i] = run;
        if (want_groups && c[j] > 0) {
          int32_t* gr = a.groups + static_cast<int64_t>(grun) * 5;
          const int64_t bh = i / a.nb;
          gr[0] = static_cast<int>(bh / a.H);
          gr[1] = static_cast<int>(bh % a.H);
          gr[2] = static_cast<int>(i % a.nb);
          gr[3] = run;
          gr[4] = c[j];
          ++grun;
        }
        run += c[j];
      }
    }
    carry += total;
    gcarry += gtotal;
  }
  if (threadIdx.x == 0) {
    ptr[n] = carry;
    // meta = {nnz, G, 0, ...}; the transposed CSR holds nnz entries too
    if (kind == 0) {
      a.meta[0] = carry;
      a.meta[1] = gcarry;
    }
  }
}

// Small masks, row lists only: one CTA stages the whole mask in shared memory with coalesced
// independent loads, then counts, scans and fills from there in a single launch (the launch
// latencies and dependent global reads of the general path cost more than the work itself here).
constexpr int kSmallRows = 4096;
constexpr int kSmallBytes = 160 * 1024;

__global__ void __launch_bounds__(kScanThreads) lists_rows_small_kernel(const ListArgs a) {
  extern __shared__ __align__(16) uint8_t s_mask[];  // rows * nb bytes, row-major
  __shared__ int s_cnt[kSmallRows];
  __shared__ int s_warp[33];
  const int rows = a.B * a.H * a.nb;
  const int total = rows * a.nb;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool contiguous = a.s3 == 1 && a.s2 == a.nb && (a.H == 1 || a.s1 == a.nb * a.nb) &&
                          (a.B == 1 || a.s0 == static_cast<int64_t>(a.H) * a.nb * a.nb) &&
                          (reinterpret_cast<uintptr_t>(a.block) & 15) == 0;
  if (contiguous) {
    const uint4* src = reinterpret_cast<const uint4*>(a.block);
    uint4* dst = reinterpret_cast<uint4*>(s_mask);
    for (int i = threadIdx.x; i < total / 16; i += kScanThreads) dst[i] = __ldg(src + i);
    for (int i = (total / 16) * 16 + threadIdx.x; i < total; i += kScanThreads)
      s_mask[i] = a.block[i];
  } else {
    for (int i = threadIdx.x; i < total; i += kScanThreads) {
      const int r = i / a.nb, c = i - r * a.nb;
      const int bh = r / a.nb, m = r - bh * a.nb;
      s_mask[i] = a.block[(bh / a.H) * a.s0 + (bh % a.H) * a.s1 + m * a.s2 + c * a.s3];
    }
  }
  __syncthreads();
  for (int r = warp; r < rows; r += kScanThreads / 32) {
    const uint8_t* row = s_mask + r * a.nb;
    int count = 0;
    for (int c0 = 0; c0 < a.nb; c0 += 32) {
      const int c = c0 + lane;
      const bool f = c < a.nb && row[c] != 0;
      count += __popc(__ballot_sync(0xffffffffu, f));
    }
    if (lane == 0) s_cnt[r] = count;
  }
  __syncthreads();
  constexpr int kPer = kSmallRows / kScanThreads;
  const int i0 = threadIdx.x * kPer;
  int sum = 0, nonempty = 0;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int c = (i0 + i < rows) ? s_cnt[i0 + i] : 0;
    sum += c;
    nonempty += c > 0;
  }
  int total_nnz = 0, gtotal = 0;
  int run = block_exclusive_scan(sum, s_warp, &total_nnz);
  int grun = block_exclusive_scan(nonempty, s_warp, &gtotal);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int r = i0 + i;
    if (r < rows) {
      const int c = s_cnt[r];
      s_cnt[r] = run;
      a.ptr[0][r] = run;
      if (a.groups != nullptr && c > 0) {
        int32_t* gr = a.groups + static_cast<int64_t>(grun) * 5;
        const int bh = r / a.nb;
        gr[0] = bh / a.H;
        gr[1] = bh % a.H;
        gr[2] = r % a.nb;
        gr[3] = run;
        gr[4] = c;
        ++grun;
      }
      run += c;
    }
  }
  if (threadIdx.x == 0) {
    a.ptr[0][rows] = total_nnz;
    a.meta[0] = total_nnz;
    a.meta[1] = gtotal;
  }
  if (threadIdx.x >= 2 && threadIdx.x < 8) a.meta[threadIdx.x] = 0;
  __syncthreads();
  for (int r = warp; r < rows; r += kScanThreads / 32) {
    const uint8_t* row = s_mask + r * a.nb;
    int32_t* out = a.ent[0] + s_cnt[r];
    int count = 0;
    for (int c0 = 0; c0 < a.nb; c0 += 32) {
      const int c = c0 + lane;
      const int byte = c < a.nb ? row[c] : 0;
      const bool f = byte != 0;
      const unsigned mk = __ballot_sync(0xffffffffu, f);
      if (f) out[count + __popc(mk & ((1u << lane) - 1u))] = list_entry(c, byte);
      count += __popc(mk);
    }
  }
}

}  // namespace bsa

extern "C" int bsa_mask_reduce(const uint8_t* dense, const int64_t s[4], int B, int H, int N,
                               uint8_t* block, int32_t* partial_tiles, int mark_partial,
                               void* stream) {
  using namespace bsa;
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0) return BSA_ERR_BAD_SHAPE;
  if (!dense || !block || !is_aligned(dense, 16)) return BSA_ERR_BAD_POINTER;
  if (s[3] != 1 || s[2] <= 0 || (s[2] % 16) != 0 || s[0] < 0 || s[1] < 0 || (s[0] % 16) != 0 ||
      (s[1] % 16) != 0)
    return BSA_ERR_BAD_STRIDE;
  const int nb = N / kBlock;
  if (static_cast<int64_t>(B) * H > 65535 || nb > 65535) return BSA_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (partial_tiles && cudaMemsetAsync(partial_tiles, 0, sizeof(int32_t), st) != cudaSuccess)
    return BSA_ERR_CUDA;
  const dim3 grid((N + kReduceCols - 1) / kReduceCols, nb, B * H);
  mask_reduce_kernel<<<grid, kReduceThreads, 0, st>>>(dense, s[0], s[1], s[2], H, N, nb, block,
                                                      partial_tiles, mark_partial);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}

extern "C" int bsa_tile_list_sizes(int B, int H, int nb, bsa_list_sizes* out) {
  if (B <= 0 || H <= 0 || nb <= 0 || !out) return BSA_ERR_BAD_SHAPE;
  const int64_t rows = static_cast<int64_t>(B) * H * nb;
  out->row_ptr = rows + 1;
  out->col_idx = rows * nb;
  out->col_ptr = rows + 1;
  out->row_idx = rows * nb;
  out->groups = rows * 5;
  out->meta = 8;
  return BSA_OK;
}

extern "C" int bsa_tile_lists_build(const uint8_t* block, const int64_t s[4], int B, int H, int nb,
                                    int32_t* row_ptr, int32_t* col_idx, int32_t* col_ptr,
                                    int32_t* row_idx, int32_t* groups, int32_t* meta,
                                    void* stream) {
  using namespace bsa;
  if (B <= 0 || H <= 0 || nb <= 0) return BSA_ERR_BAD_SHAPE;
  if (!block || !meta) return BSA_ERR_BAD_POINTER;
  if ((row_ptr == nullptr) != (col_idx == nullptr) || (col_ptr == nullptr) != (row_idx == nullptr) ||
      (groups != nullptr && row_ptr == nullptr))
    return BSA_ERR_BAD_POINTER;
  for (int i = 0; i < 4; ++i)
    if (s[i] < 0) return BSA_ERR_BAD_STRIDE;
  // entry offsets are int32: the worst-case entry count must fit
  if (static_cast<int64_t>(B) * H * nb * nb > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  ListArgs a;
  a.block = block;
  a.s0 = s[0];
  a.s1 = s[1];
  a.s2 = s[2];
  a.s3 = s[3];
  a.B = B;
  a.H = H;
  a.nb = nb;
  a.ptr[0] = row_ptr;
  a.ent[0] = col_idx;
  a.ptr[1] = col_ptr;
  a.ent[1] = row_idx;
  a.groups = groups;
  a.meta = meta;

  const int64_t bh = static_cast<int64_t>(B) * H;
  const int64_t warps_per_cta = kListThreads / 32;
  int64_t blocks = 1;
  auto upd = [&](int64_t v) { blocks = v > blocks ? v : blocks; };
  if (row_ptr) upd((bh * nb + warps_per_cta - 1) / warps_per_cta);
  if (col_ptr) upd(bh * ((nb + 31) / 32));
  if (blocks > 0x7fffffffLL) return BSA_ERR_TOO_LARGE;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (row_ptr && !col_ptr && bh * nb <= kSmallRows &&
      bh * nb * nb <= kSmallBytes) {
    const size_t smem = static_cast<size_t>((bh * nb * nb + 15) & ~15LL);
    int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(lists_rows_small_kernel),
                                 kSmallBytes);
    if (rc != BSA_OK) return rc;
    lists_rows_small_kernel<<<1, kScanThreads, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
  }
  if (cudaMemsetAsync(meta, 0, 8 * sizeof(int32_t), st) != cudaSuccess) return BSA_ERR_CUDA;
  const dim3 grid(static_cast<unsigned>(blocks), 2);
  lists_pass_kernel<false><<<grid, kListThreads, 0, st>>>(a);
  lists_scan_kernel<<<2, kScanThreads, 0, st>>>(a);
  lists_pass_kernel<true><<<grid, kListThreads, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}
