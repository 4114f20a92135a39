// Forward attention straight from a block mask for callers that must not allocate device memory.
//
// The ordinary path needs two caller-provided device buffers between its steps: the CSR row lists
// (row_ptr, col_idx) that bsa_tile_lists_build writes and bsa_attn_fwd reads.  Some hosts cannot
// provide them at call time: an inference-engine plugin whose workspace size was fixed when the
// engine was built, or a process whose device memory is already handed out in full to another
// pool, so that a driver allocation would fail or stall the device.  For them this file keeps the
// lists in a fixed device array that is part of the library image.
#include <atomic>

#include "host_common.h"

namespace {

// int32 words: meta[8] | row_ptr[rows + 1] | col_idx[rows * nb]  (see the capacity check below).
// Every GPU that loads the library holds this array until the process exits.
constexpr int64_t kStaticScratchInts = BSA_STATIC_SCRATCH_INTS;
static __device__ __align__(256) int32_t g_static_lists[kStaticScratchInts];

// The array's name is only a host-side handle; kernels need its device address, which differs per
// device.  Looked up once per device, with that device current; with lazy module loading this
// look-up is also what makes the driver load the module and reserve the array on the device.
int32_t* static_lists_for_current_device(int* status) {
  static std::atomic<int32_t*> cached[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *status = BSA_ERR_CUDA;
    return nullptr;
  }
  int32_t* p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_static_lists) != cudaSuccess || addr == nullptr) {
      (void)cudaGetLastError();
      *status = BSA_ERR_CUDA;
      return nullptr;
    }
    p = static_cast<int32_t*>(addr);
    cached[dev].store(p, std::memory_order_release);
  }
  *status = BSA_OK;
  return p;
}

}  // namespace

extern "C" int bsa_attn_fwd_block_mask_static(
    const void* q, const int64_t q_strides[4], const void* k, const int64_t k_strides[4],
    const void* v, const int64_t v_strides[4], void* o, const int64_t o_strides[4], float* lse2,
    const uint8_t* block, const int64_t block_strides[4], int Bm, int Hm, float sm_scale,
    int dtype, int B, int H, int N, int D, void* stream) {
  using namespace bsa;
  if (B <= 0 || H <= 0 || N <= 0 || (N % kBlock) != 0 || D != kHeadDim) return BSA_ERR_BAD_SHAPE;
  if ((Bm != 1 && Bm != B) || (Hm != 1 && Hm != H)) return BSA_ERR_BAD_SHAPE;
  if (!block || !block_strides) return BSA_ERR_BAD_POINTER;
  const int64_t nb = N / kBlock;
  const int64_t rows = static_cast<int64_t>(Bm) * Hm * nb;
  // worst case: every block of every mask row is kept
  if (8 + (rows + 1) + rows * nb > kStaticScratchInts) return BSA_ERR_TOO_LARGE;

  int rc = BSA_OK;
  int32_t* base = static_lists_for_current_device(&rc);
  if (rc != BSA_OK) return rc;
  int32_t* meta = base;
  int32_t* row_ptr = base + 8;
  int32_t* col_idx = row_ptr + (rows + 1);

  // The builder writes every word it later reads (counts, offsets, entries, meta), so nothing of
  // the previous call's contents has to be cleared first.
  rc = bsa_tile_lists_build(block, block_strides, Bm, Hm, static_cast<int>(nb), row_ptr, col_idx,
                            nullptr, nullptr, nullptr, meta, stream);
  if (rc != BSA_OK) return rc;
  return bsa_attn_fwd(q, q_strides, k, k_strides, v, v_strides, o, o_strides, lse2, nullptr,
                      row_ptr, col_idx, Bm > 1 ? Hm : 0, Hm > 1 ? 1 : 0, sm_scale, dtype, B, H, N,
                      D, nullptr, nullptr, stream);
}

extern "C" int bsa_static_warmup(void) {
  int rc = BSA_OK;
  (void)static_lists_for_current_device(&rc);
  return rc;
}
