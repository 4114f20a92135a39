/*
 * bsattn.h — C ABI of libbsattn: 64x64 block-sparse FlashAttention-2 for NVIDIA B200 (sm_100a).
 *
 * Every entry point
 *   - takes plain device pointers, sizes and element strides (no torch types),
 *   - borrows all buffers (the caller owns inputs, outputs and workspaces),
 *   - enqueues its work on `stream` (a cudaStream_t passed as void*) of the CURRENT device and
 *     returns without synchronising,
 *   - returns BSA_OK (0) or a negative bsa_status; it never throws, exits or prints.
 *
 * The library replaces the device side of the reference's Python package `fa2_custom_mask`;
 * each declaration cites the reference interface (path:line inside the reference project)
 * whose work it takes over.
 *
 * Vocabulary: a "block" is 64 consecutive tokens; nb = N/64 blocks per sequence; a "tile" is one
 * (query block m, key block n) pair that the block mask keeps.  The kernels walk row lists (per
 * query block its kept key blocks: forward, dQ) and column lists (per key block the query blocks
 * that keep it: dK/dV).
 */
#ifndef BSATTN_H_
#define BSATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSA_VERSION 200

/* Tile-list entries (col_idx, row_idx) are block indices; an entry of a tile that is kept but has
 * masked elements inside (mask byte 2, see bsa_mask_reduce) also carries this flag. */
#define BSA_LIST_PARTIAL_FLAG (1 << 30)

typedef enum bsa_status {
  BSA_OK = 0,
  BSA_ERR_BAD_SHAPE = -1,      /* N not a multiple of 64, D != 64, non-positive sizes, bad row range,
                                  negative sm_scale                                               */
  BSA_ERR_BAD_DTYPE = -2,      /* dtype is neither BSA_F16 nor BSA_BF16                           */
  BSA_ERR_BAD_STRIDE = -3,     /* innermost stride != 1, or an outer stride not 16-byte aligned   */
  BSA_ERR_BAD_POINTER = -4,    /* null or misaligned pointer                                      */
  BSA_ERR_CUDA = -5,           /* a CUDA runtime/driver call failed (launch, attribute, tensor map) */
  BSA_ERR_NO_DRIVER = -6,      /* cuTensorMapEncodeTiled could not be resolved                    */
  BSA_ERR_UNSUPPORTED_ARCH = -7, /* current device is not compute capability 10.x                 */
  BSA_ERR_TOO_LARGE = -8,      /* problem exceeds a documented fixed capacity                     */
  BSA_ERR_DEVICE_TIMEOUT = -9  /* reported by bsa_check_status: a bounded device wait gave up     */
} bsa_status;

typedef enum bsa_dtype { BSA_F16 = 0, BSA_BF16 = 1 } bsa_dtype;

/* Library version (BSA_VERSION of the build). No reference counterpart. */
int bsa_version(void);

/* Static, human-readable text for a bsa_status. No reference counterpart
 * (the reference raises Python AssertionErrors: fa2_custom_mask/fa2_custom_mask.py:57-58,99-100,113). */
const char* bsa_strerror(int status);

/*
 * Dense boolean mask -> block mask.  block[b,h,i,j] = any(dense[b,h,64i:64i+64, 64j:64j+64]).
 * Inverse of the expansion the reference uses for its naive check (kernel-test.py:18); the
 * reference's op itself only accepts the block mask (fa2_custom_mask/fa2_custom_mask.py:17-21).
 *   dense    : bytes (0 = masked, non-zero = kept), logical shape [B,H,N,N], element strides
 *              dense_strides[4] (0 allowed for broadcast over b/h); last stride must be 1, the
 *              row stride and base address multiples of 16.
 *   block    : out, contiguous [B,H,nb,nb] bytes: 0 = no element kept, 1 = kept.  With
 *              mark_partial != 0 a tile that is kept but also has masked elements gets 2, which
 *              the list builder and the forward/backward kernels understand: given the dense
 *              mask as well, they apply it element by element inside those tiles (the in-tile
 *              mask the reference sketches in fa2_custom_mask/fa2_fwd.py:57-75 and its naive
 *              check applies, kernel-test.py:37-40).
 *   partial_tiles : optional out (may be NULL), one int32 that the call first zeroes and then
 *              increments once per tile that is neither all-kept nor all-masked.
 */
int bsa_mask_reduce(const uint8_t* dense, const int64_t dense_strides[4], int B, int H, int N,
                    uint8_t* block, int32_t* partial_tiles, int mark_partial, void* stream);

/* Number of int32 elements the caller must provide for each output of bsa_tile_lists_build. */
typedef struct bsa_list_sizes {
  int64_t row_ptr;    /* B*H*nb + 1                        */
  int64_t col_idx;    /* worst case B*H*nb*nb              */
  int64_t col_ptr;    /* B*H*nb + 1                        */
  int64_t row_idx;    /* worst case B*H*nb*nb              */
  int64_t groups;     /* worst case 5*B*H*nb               */
  int64_t meta;       /* 8                                 */
} bsa_list_sizes;
int bsa_tile_list_sizes(int B, int H, int nb, bsa_list_sizes* out);

/*
 * Block mask -> tile lists, all built on the device with no host synchronisation.
 * Replaces build_groups_from_block_mask (fa2_custom_mask/fa2_custom_mask.py:15-38), whose
 * outputs are reproduced bit-exactly:  n_list == col_idx[0:nnz]  and  groups == groups[0:G].
 *   block      : bytes (0, 1 or 2, see bsa_mask_reduce), logical [B,H,nb,nb], element strides
 *                block_strides[4] (0 = broadcast).  Entries of tiles with byte 2 carry
 *                BSA_LIST_PARTIAL_FLAG; a mask of zeros and ones gives the reference's lists.
 *   row_ptr/col_idx : CSR over rows r=(b*H+h)*nb+m, empty rows kept, columns ascending
 *                     (forward and dQ kernels).
 *   col_ptr/row_idx : CSR of the transposed mask (per key block, query blocks ascending;
 *                     dK/dV kernel).
 *   groups     : rows (b,h,m,start,len) of the non-empty rows only, in row order.
 *   meta       : int32[8] = {nnz, G, 0,0,0,0,0,0}.
 * Any (ptr,idx) pair, and groups, may be NULL to skip that product; meta is required.
 */
int bsa_tile_lists_build(const uint8_t* block, const int64_t block_strides[4], int B, int H, int nb,
                         int32_t* row_ptr, int32_t* col_idx, int32_t* col_ptr, int32_t* row_idx,
                         int32_t* groups, int32_t* meta, void* stream);

/*
 * Forward attention over the listed tiles; replaces the _attn_fwd launch
 * (fa2_custom_mask/fa2_custom_mask.py:77-87, kernel fa2_custom_mask/fa2_fwd.py:108-206).
 *   q,k,v,o : [B,H,N,64] fp16/bf16, element strides *_strides[4]; last stride 1, others multiples
 *             of 8 elements, base 16-byte aligned.
 *   sm_scale: the factor on Q K^T; must not be negative (the kernel takes row maxima before
 *             scaling).
 *   lse2    : out fp32 [B,H,N] contiguous: log2-sum-exp2 of the scaled logits
 *             (natural-log LSE = lse2 * ln 2); -inf for rows of query blocks with no listed tile.
 *   rowmax  : optional out fp32 [B,H,N] (may be NULL): running row maximum of the scaled logits in
 *             the exp2 domain, the quantity the reference stores in its `M` buffer
 *             (fa2_custom_mask/fa2_fwd.py:193-196).
 *   row_ptr/col_idx : CSR row lists from bsa_tile_lists_build built for a mask of shape
 *             [Bm,Hm,nb,nb]; list_b_stride/list_h_stride give the list index of head (b,h) as
 *             b*list_b_stride + h*list_h_stride (0 for a broadcast axis).
 *   Rows of query blocks without any listed tile get o = 0 (the reference leaves them unwritten).
 *   work_counter : optional int32 device word (may be NULL).  The kernel is persistent (one CTA
 *             per SM); with a counter the CTAs draw query blocks from it as they become free, which
 *             evens out rows of unequal length; without one every CTA walks a fixed stride of
 *             query blocks.  The word must hold 0 when the kernel starts and holds 0 again when it
 *             ends, so one zeroed word serves any number of calls that cannot overlap on the GPU
 *             (calls on one stream); calls that may overlap need a word each.  A CTA whose bounded
 *             wait gave up still draws its remaining tickets, so the word returns to 0 then too.
 *   status  : optional int32 word (may be NULL) in device memory or in pinned host memory that the
 *             device can reach; a non-zero value after the stream drains
 *             means a bounded wait inside the kernel gave up (see bsa_check_status).
 */
int bsa_attn_fwd(const void* q, const int64_t q_strides[4], const void* k,
                 const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* o,
                 const int64_t o_strides[4], float* lse2, float* rowmax, const int32_t* row_ptr,
                 const int32_t* col_idx, int list_b_stride, int list_h_stride, float sm_scale,
                 int dtype, int B, int H, int N, int D, int32_t* work_counter, int32_t* status,
                 void* stream);

/*
 * The same forward with the list building fused in: every CTA lists the kept key blocks of its own
 * mask row, so no tile lists (and no list kernel) are needed for a forward-only call.  Replaces
 * build_groups_from_block_mask + the _attn_fwd launch together
 * (fa2_custom_mask/fa2_custom_mask.py:48 and :77-87).
 *   block : bytes, logical [Bm,Hm,nb,nb] with element strides block_strides[4]; Bm is 1 or B, Hm is
 *           1 or H.  Other arguments and results as in bsa_attn_fwd.  Both forward entry points
 *           need N <= 131072.
 */
int bsa_attn_fwd_block_mask(const void* q, const int64_t q_strides[4], const void* k,
                            const int64_t k_strides[4], const void* v, const int64_t v_strides[4],
                            void* o, const int64_t o_strides[4], float* lse2, float* rowmax,
                            const uint8_t* block, const int64_t block_strides[4], int Bm, int Hm,
                            float sm_scale, int dtype, int B, int H, int N, int D,
                            int32_t* work_counter, int32_t* status, void* stream);

/*
 * The two forward entry points in their general form.
 *   row_begin, row_end : only the query-block rows [row_begin, row_end) of every (batch, head) are
 *           computed; rows of o, lse2 and rowmax outside the range are not touched.  The reference
 *           launches one program per listed (batch, head, query block) row
 *           (fa2_custom_mask/fa2_custom_mask.py:69-70), so any subset of its grid is a valid
 *           launch; this is the same freedom, used to split the rows of a head across GPUs when
 *           there are fewer (batch, head) units than GPUs (every GPU then holds all of that
 *           head's K and V).  An empty range returns BSA_OK without launching.
 *   dense, dense_strides : optional (may be NULL) element-level mask, bytes, logical [B,H,N,N]
 *           with element strides dense_strides[4] (0 for a broadcast axis; last stride 1, base and
 *           the other strides multiples of 16).  Tiles marked 2 in `block` (flagged in the lists)
 *           then keep only the elements whose byte is non-zero; rows without any kept element
 *           get o = 0 and lse2 = -inf.  Without it every listed tile is attended in full, as in
 *           the reference kernel.
 * bsa_attn_fwd / bsa_attn_fwd_block_mask are these with the range [0, N/64) and no dense mask.
 */
int bsa_attn_fwd_rows(const void* q, const int64_t q_strides[4], const void* k,
                      const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* o,
                      const int64_t o_strides[4], float* lse2, float* rowmax,
                      const int32_t* row_ptr, const int32_t* col_idx, int list_b_stride,
                      int list_h_stride, float sm_scale, int dtype, int B, int H, int N, int D,
                      int row_begin, int row_end, const uint8_t* dense,
                      const int64_t dense_strides[4], int32_t* work_counter, int32_t* status,
                      void* stream);
int bsa_attn_fwd_block_mask_rows(const void* q, const int64_t q_strides[4], const void* k,
                                 const int64_t k_strides[4], const void* v,
                                 const int64_t v_strides[4], void* o, const int64_t o_strides[4],
                                 float* lse2, float* rowmax, const uint8_t* block,
                                 const int64_t block_strides[4], int Bm, int Hm, float sm_scale,
                                 int dtype, int B, int H, int N, int D, int row_begin, int row_end,
                                 const uint8_t* dense, const int64_t dense_strides[4],
                                 int32_t* work_counter, int32_t* status, void* stream);

/*
 * delta[b,h,i] = sum_d o[b,h,i,d] * do[b,h,i,d] in fp32; replaces _attn_bwd_preprocess
 * (fa2_custom_mask/fa2_bwd.py:5-19, launch fa2_custom_mask/fa2_custom_mask.py:114-121).
 * o and do share o_strides; delta is contiguous [B,H,N].
 */
int bsa_attn_bwd_delta(const void* o, const void* dout, const int64_t o_strides[4], float* delta,
                       int dtype, int B, int H, int N, int D, void* stream);

/*
 * dK and dV; replaces _attn_bwd_dkdv
 * (fa2_custom_mask/fa2_bwd.py:23-81, driven from fa2_custom_mask/fa2_bwd.py:199-234).
 * All of q,k,v,dout,dk,dv share `strides`.  lse2 and delta are the outputs of bsa_attn_fwd and
 * bsa_attn_bwd_delta.  col_ptr/row_idx are the column lists of bsa_tile_lists_build (for every key
 * block the query blocks that list it), addressed like the row lists of bsa_attn_fwd.  Key blocks
 * that no query block lists get dk = dv = 0.  work_counter: as in bsa_attn_fwd (both backward
 * kernels are persistent too; the same zeroed word can serve all calls of one stream).
 * dense, dense_strides: the optional element-level mask of bsa_attn_fwd_rows (NULL = none), applied
 * inside the tiles whose list entries carry BSA_LIST_PARTIAL_FLAG; pass what the forward was given.
 */
int bsa_attn_bwd_dkdv(const void* q, const void* k, const void* v, const void* dout,
                      const int64_t strides[4], const float* lse2, const float* delta, void* dk,
                      void* dv, const int32_t* col_ptr, const int32_t* row_idx,
                      int list_b_stride, int list_h_stride, float sm_scale, int dtype, int B, int H,
                      int N, int D, const uint8_t* dense, const int64_t dense_strides[4],
                      int32_t* work_counter, int32_t* status, void* stream);

/*
 * dQ over the row lists (row_ptr/col_idx, as in bsa_attn_fwd); replaces _attn_bwd_dq
 * (fa2_custom_mask/fa2_bwd.py:85-137, driven from fa2_custom_mask/fa2_bwd.py:237-285).
 */
int bsa_attn_bwd_dq(const void* q, const void* k, const void* v, const void* dout,
                    const int64_t strides[4], const float* lse2, const float* delta, void* dq,
                    const int32_t* row_ptr, const int32_t* col_idx, int list_b_stride,
                    int list_h_stride, float sm_scale, int dtype, int B, int H, int N, int D,
                    const uint8_t* dense, const int64_t dense_strides[4], int32_t* work_counter,
                    int32_t* status, void* stream);

/*
 * Head-wise token reorder; replaces reorder_kernel (fa2_custom_mask/permute.py:5-58, launched from
 * fa2_custom_mask/functional.py:5-20).  For every head h with order (p0,p1,p2) = orders[3h..3h+2],
 * a token at grid coordinate (f,y,x) of the F x Hh x W grid moves to the position it has when the
 * grid axes are laid out in the order (p0,p1,p2).
 *   in/out : [B,heads,T=F*Hh*W,D] with element strides `strides` (shared by in and out, as in the
 *            reference); elem_bytes is 1, 2, 4 or 8.
 *   orders : device int32 [heads,3].  A row that is not a permutation of (0,1,2) leaves that
 *            head's rows of `out` unwritten (checked on the device, no error is reported).
 */
int bsa_reorder(const void* in, void* out, const int64_t strides[4], const int32_t* orders, int B,
                int heads, int T, int D, int F, int Hh, int W, int elem_bytes, void* stream);

/*
 * Inverse of bsa_reorder; replaces inv_reorder_kernel (fa2_custom_mask/permute.py:60-126, launched
 * from fa2_custom_mask/functional.py:46-62).  `orders` is the forward order that produced `in`,
 * `inv_orders` its inverse-order table row per head, exactly as the reference passes them.
 */
int bsa_inv_reorder(const void* in, void* out, const int64_t strides[4], const int32_t* orders,
                    const int32_t* inv_orders, int B, int heads, int T, int D, int F, int Hh, int W,
                    int elem_bytes, void* stream);

/*
 * The same two gathers with separate element strides for `in` and `out` (last stride 1 in both).
 * The reference's kernels share one stride set, so its wrappers first copy the image-token slice
 * of q, k, v to a contiguous tensor (fa2_custom_mask/functional.py:35-37, 82); with these entry
 * points the slice is read where it lies and that copy disappears.  `in` and `out` must not
 * overlap.
 */
int bsa_reorder_strided(const void* in, const int64_t in_strides[4], void* out,
                        const int64_t out_strides[4], const int32_t* orders, int B, int heads, int T,
                        int D, int F, int Hh, int W, int elem_bytes, void* stream);
int bsa_inv_reorder_strided(const void* in, const int64_t in_strides[4], void* out,
                            const int64_t out_strides[4], const int32_t* orders,
                            const int32_t* inv_orders, int B, int heads, int T, int D, int F, int Hh,
                            int W, int elem_bytes, void* stream);

/*
 * Forward attention directly from a block mask, allocating nothing.  It has no counterpart in the
 * reference; it exists for hosts that cannot hand the library device buffers at call time, such as
 * an inference-engine plugin whose workspace was sized when the engine was built, or a process
 * whose device memory already belongs in full to another pool.  The row lists that
 * bsa_tile_lists_build would write into caller memory go into a fixed array inside the library
 * image instead (BSA_STATIC_SCRATCH_INTS 32-bit words, held by every GPU that loads the library
 * until the process exits); the result equals bsa_tile_lists_build followed by bsa_attn_fwd.
 *   block : bytes, logical [Bm,Hm,nb,nb] with element strides block_strides[4]; Bm is 1 or B, Hm is
 *           1 or H.  All other arguments as in bsa_attn_fwd.  rowmax, the work counter and the
 *           status word are not offered here: the query blocks are handed out at a fixed stride
 *           (a few percent slower than the counter on masks with rows of unequal length), and a
 *           bounded wait that gave up is not reported.
 * Limit: 8 + Bm*Hm*nb + 1 + Bm*Hm*nb*nb <= BSA_STATIC_SCRATCH_INTS, else BSA_ERR_TOO_LARGE
 * (one shared mask up to N = 92,000; eight per-head masks up to N = 32,000).
 * The first call on each device looks up the array's device address.  With CUDA's lazy module
 * loading that is also the moment the driver loads the library's kernels onto the device and
 * reserves the array's 8 MiB there, so make that first call (or call bsa_static_warmup) early:
 * before the process hands the rest of the device memory to its own pool, and outside any stream
 * capture.  After that, a call makes no cudaMalloc/cudaFree and calls no allocating library
 * routine.  The looked-up address is remembered per device for the life of the process: a
 * cudaDeviceReset invalidates it.
 * All calls on a device share the one array: two calls whose GPU work may overlap (different
 * streams, or different host threads) race on it and must be serialised by the caller.
 */
#define BSA_STATIC_SCRATCH_INTS (2 * 1024 * 1024)
int bsa_attn_fwd_block_mask_static(const void* q, const int64_t q_strides[4], const void* k,
                                   const int64_t k_strides[4], const void* v,
                                   const int64_t v_strides[4], void* o, const int64_t o_strides[4],
                                   float* lse2, const uint8_t* block,
                                   const int64_t block_strides[4], int Bm, int Hm, float sm_scale,
                                   int dtype, int B, int H, int N, int D, void* stream);

/*
 * Does only the first-call set-up of bsa_attn_fwd_block_mask_static on the current device (module
 * load, address look-up) and enqueues nothing.  No reference counterpart.
 */
int bsa_static_warmup(void);

/*
 * Synchronises `stream`, reads the device status word and returns BSA_OK, BSA_ERR_DEVICE_TIMEOUT
 * or BSA_ERR_CUDA.  No reference counterpart.
 */
int bsa_check_status(const int32_t* status, void* stream);

/*
 * Self-test of the kernels' bounded waits; no reference counterpart.  Launches one small CTA in
 * which one warp waits on a barrier that nothing ever completes and a second warp waits beside
 * it.  The first wait runs out after the library's wait limit (about two seconds), records 99 in
 * `status` (optional) and raises the CTA's give-up flag, which releases the second warp; both
 * leave through the end of the kernel.  `report` (device, 4 x int32) receives: [0] 1 if the first
 * wait was satisfied (never), [1] the same for the second, [2] 1 once both warps reached the end
 * of the kernel, [3] milliseconds spent.  The context stays usable; bsa_check_status on the same
 * word then returns BSA_ERR_DEVICE_TIMEOUT.
 */
int bsa_selftest_bounded_wait(int32_t* status, int32_t* report, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BSATTN_H_ */
