#include "host_common.h"

#include <atomic>

namespace bsa {

int check_device_sm100() {
  static std::atomic<int> cached[64];  // 0 unknown, 1 ok, 2 unsupported
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return BSA_ERR_CUDA;
  if (dev >= 0 && dev < 64) {
    int c = cached[dev].load(std::memory_order_relaxed);
    if (c == 1) return BSA_OK;
    if (c == 2) return BSA_ERR_UNSUPPORTED_ARCH;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return BSA_ERR_CUDA;
  const bool ok = (major == 10);
  if (dev >= 0 && dev < 64) cached[dev].store(ok ? 1 : 2, std::memory_order_relaxed);
  return ok ? BSA_OK : BSA_ERR_UNSUPPORTED_ARCH;
}

int check_qkv_operand(const void* p, const int64_t s[4]) {
  if (p == nullptr || !is_aligned(p, 16)) return BSA_ERR_BAD_POINTER;
  if (s[3] != 1) return BSA_ERR_BAD_STRIDE;
  for (int i = 0; i < 3; ++i)
    if (s[i] <= 0 || (s[i] % 8) != 0) return BSA_ERR_BAD_STRIDE;
  return BSA_OK;
}

int sm_count(int* out) {
  static std::atomic<int> cached[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return BSA_ERR_CUDA;
  int n = (dev >= 0 && dev < 64) ? cached[dev].load(std::memory_order_relaxed) : 0;
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return BSA_ERR_CUDA;
    if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  }
  *out = n;
  return BSA_OK;
}

int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  // a handful of kernels x devices: a small fixed table guarded by a spin flag is enough
  struct Entry { const void* k; int dev; };
  static Entry table[128];
  static std::atomic<int> count{0};
  static std::atomic_flag lock = ATOMIC_FLAG_INIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return BSA_ERR_CUDA;
  const int n = count.load(std::memory_order_acquire);
  for (int i = 0; i < n; ++i)
    if (table[i].k == kernel && table[i].dev == dev) return BSA_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(bytes)) != cudaSuccess) {
    (void)cudaGetLastError();
    return BSA_ERR_CUDA;
  }
  while (lock.test_and_set(std::memory_order_acquire)) {
  }
  const int m = count.load(std::memory_order_relaxed);
  if (m < 128) {
    table[m] = Entry{kernel, dev};
    count.store(m + 1, std::memory_order_release);
  }
  lock.clear(std::memory_order_release);
  return BSA_OK;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn resolve_encode() {
  static std::atomic<void*> cached{nullptr};
  void* fn = cached.load(std::memory_order_acquire);
  if (fn) return reinterpret_cast<encode_tiled_fn>(fn);
  cudaDriverEntryPointQueryResult qres;
  void* sym = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  cached.store(sym, std::memory_order_release);
  return reinterpret_cast<encode_tiled_fn>(sym);
}

int make_qkv_tmap(CUtensorMap* out, const void* base, const int64_t s[4], int B, int H, int N,
                  int dtype, int box_rows) {
  encode_tiled_fn enc = resolve_encode();
  if (!enc) return BSA_ERR_NO_DRIVER;
  const CUtensorMapDataType dt =
      dtype == BSA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // innermost first: (d, n, h, b)
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(N),
                        static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s[2]) * 2, static_cast<cuuint64_t>(s[1]) * 2,
                           static_cast<cuuint64_t>(s[0]) * 2};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(kHeadDim), static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BSA_OK : BSA_ERR_CUDA;
}

}  // namespace bsa

extern "C" int bsa_version(void) { return BSA_VERSION; }

extern "C" const char* bsa_strerror(int status) {
  switch (status) {
    case BSA_OK: return "ok";
    case BSA_ERR_BAD_SHAPE: return "bad shape (N must be a positive multiple of 64, D must be 64)";
    case BSA_ERR_BAD_DTYPE: return "bad dtype (fp16 or bf16 only)";
    case BSA_ERR_BAD_STRIDE:
      return "bad stride (innermost stride must be 1, outer strides multiples of 16 bytes)";
    case BSA_ERR_BAD_POINTER: return "null or misaligned pointer";
    case BSA_ERR_CUDA: return "a CUDA call failed";
    case BSA_ERR_NO_DRIVER: return "cuTensorMapEncodeTiled could not be resolved from the driver";
    case BSA_ERR_UNSUPPORTED_ARCH: return "current device is not compute capability 10.x (B200)";
    case BSA_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point";
    case BSA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    default: return "unknown status";
  }
}

extern "C" int bsa_check_status(const int32_t* status, void* stream) {
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return BSA_ERR_CUDA;
  if (status == nullptr) return BSA_OK;
  int32_t host = 0;
  if (cudaMemcpy(&host, status, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess)
    return BSA_ERR_CUDA;
  return host == 0 ? BSA_OK : BSA_ERR_DEVICE_TIMEOUT;
}
