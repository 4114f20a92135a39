// Host-side helpers shared by the entry points: argument checks, per-device set-up, and TMA
// tensor-map encoding through a driver entry point resolved at run time (the library does not
// link libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bsattn.h"

namespace bsa {

constexpr int kBlock = 64;     // tokens per mask block (semantic: the reference's BLOCK_M = BLOCK_N)
constexpr int kHeadDim = 64;   // supported head dimension

inline bool is_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// 0 when the current device is compute capability 10.x, else a negative status.
int check_device_sm100();

// Validates a [B,H,N,64] 16-bit operand for TMA: base 16-byte aligned, last stride 1, the other
// strides positive multiples of 8 elements.
int check_qkv_operand(const void* p, const int64_t s[4]);

// Encodes a 4-D tile map over a [B,H,N,64] 16-bit tensor with element strides s[4]:
// box = box_rows x 64 elements, 128-byte swizzle, out-of-range rows read as zero.
int make_qkv_tmap(CUtensorMap* out, const void* base, const int64_t s[4], int B, int H, int N,
                  int dtype, int box_rows);

// Number of SMs of the current device (cached per device).
int sm_count(int* out);

// Raises a kernel's dynamic shared-memory limit; done once per (kernel, device) and remembered.
int ensure_dynamic_smem(const void* kernel, size_t bytes);

}  // namespace bsa
