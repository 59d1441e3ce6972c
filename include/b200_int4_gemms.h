/*
 * C ABI of the B200 (sm_100a) quantized-GEMM library: libb200_int4_gemms.so.
 *
 * This is the boundary a host language binds (ctypes, cgo, JNI ...).  It replaces the
 * reference's HIP code-object dispatcher, native/src/dispatch.cpp, whose eight exported
 * symbols are listed beside their counterparts below.  Differences in kind, not in spirit:
 *
 *   - the kernels are linked into the library, so there is no code-object path / symbol
 *     argument, and grid / block / shared-memory sizes are decided inside the library
 *     instead of being read from per-kernel JSON by the caller;
 *   - a kernel is named by a plain-old-data variant record (dtype, layout, scale mode,
 *     epilogue, output type) instead of by a file name.
 *
 * Conventions shared with the reference (dispatch.cpp:18-23, :206-222, :224-283):
 *   - every entry point returns 0 on success and 1 on failure;
 *   - on failure a thread-local message is available from b200_int4_gemms_last_error();
 *     it is cleared on entry to every launch call;
 *   - all buffers are caller-owned DEVICE pointers; launches are asynchronous on the
 *     caller's stream (a cudaStream_t passed as an integer); no call synchronises;
 *   - the device is selected per call (cudaSetDevice(device_index)).
 *
 * Operand format (bit-exact with the reference's quant.py:32-51):
 *   int4 operands are uint8 bytes holding two signed nibbles packed along K: the low
 *   nibble is the even k index, the high nibble the odd one.  int8 operands are plain
 *   signed bytes.  Scales are bfloat16.  Accumulation is exact int32.
 */
#ifndef B200_INT4_GEMMS_H_
#define B200_INT4_GEMMS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { B200_DTYPE_INT4 = 0, B200_DTYPE_INT8 = 1 };
/* Operand layouts: first letter A, second letter B; N = as given, T = transposed.
 *   NN: A [M, Kb]   B [Kb, N]        NT: A [M, Kb]   B [N, Kb]
 *   TN: A [Kb, M]   B [Kb, N]        TT: A [Kb, M]   B [N, Kb]
 * Kb is K bytes: K/2 (rounded up) for int4, K for int8. */
enum { B200_LAYOUT_NN = 0, B200_LAYOUT_NT = 1, B200_LAYOUT_TN = 2, B200_LAYOUT_TT = 3 };
enum { B200_SCALE_PER_CHANNEL = 0, B200_SCALE_SUBCHANNEL = 1 };
enum { B200_EPILOGUE_NONE = 0, B200_EPILOGUE_RELU2 = 1, B200_EPILOGUE_SWIGLU = 2 };
/* B200_OUT_S32 stores the raw int32 accumulators (per-channel mode only, scales ignored);
 * it exists so that callers can check the integer path bit for bit. */
enum { B200_OUT_BF16 = 0, B200_OUT_F32 = 1, B200_OUT_S32 = 2 };
/* B200_PATH_AUTO picks the tcgen05 tensor-core kernel whenever the shape and pointers
 * meet its alignment rules and the plain CUDA-core kernel otherwise; the other two
 * force one of them (B200_PATH_TCGEN05 fails when the rules are not met). */
enum { B200_PATH_AUTO = 0, B200_PATH_TCGEN05 = 1, B200_PATH_SIMT = 2 };
/* PERSISTENT: one CTA (or CTA pair) per SM (pair of SMs) walks the tile list, the epilogue of one tile
 * overlapping the mainloop of the next.  TILE_PER_CTA: one CTA (or pair) per output tile, as a plain
 * non-persistent kernel would be launched; kept for comparison, slower on anything but tiny problems. */
enum { B200_SCHEDULE_PERSISTENT = 0, B200_SCHEDULE_TILE_PER_CTA = 1 };

/* AUTO: the library pairs CTAs (clusters of two SMs, 256 x 256 tiles, tcgen05 cta_group::2) when a
 * paired kernel exists for the variant, M exceeds 128 and the 256-row tiling does not cost more waves
 * than it saves per tile; else one CTA per 128 x 256 tile.  SINGLE / PAIR force one of them (PAIR falls back to SINGLE when no paired kernel
 * exists).  Results are bit-identical either way. */
enum { B200_CTA_GROUP_AUTO = 0, B200_CTA_GROUP_SINGLE = 1, B200_CTA_GROUP_PAIR = 2 };

/* Subchannel scales only: how a dense launch adds the K-groups' contributions to the fp32 running sum.
 *   FUSED (the default): out = fma(f32(acc_g) * sa_g, sb_g, out) - the last multiply and the add share one
 *     rounding; half the CUDA-core work per accumulator element, which is what limits these kernels.
 *   REFERENCE: out += (f32(acc_g) * sa_g) * sb_g with every rounding of the reference's PyTorch math
 *     (api.py:316-324): bit-identical to it.
 * Both stay far inside the bf16 output tolerance; the integer accumulators are exact either way.
 * Grouped (ragged) launches always use the reference order. */
enum { B200_ACCUMULATE_FUSED = 0, B200_ACCUMULATE_REFERENCE = 1 };

/* Where the unpacked A operand of an int4 CTA-pair kernel lives between the unpack warps and the tensor core.
 * TMEM (per-channel scales, A stored [M, Kb]): a third less traffic through the shared-memory pipe, but a single
 * accumulator buffer, so the epilogue of a tile is not hidden behind the next tile's MMAs.  AUTO picks TMEM for
 * long reductions (K >= 6144), shared memory otherwise; SMEM / TMEM force one (TMEM falls back to shared memory
 * where no such kernel exists).  Bit-identical results. */
enum { B200_A_OPERAND_AUTO = 0, B200_A_OPERAND_SMEM = 1, B200_A_OPERAND_TMEM = 2 };

/* Balanced tail of dense per-channel launches.  When the last wave of the persistent grid fills at most half of the
 * CTAs (CTA pairs), its tiles can be cut along K into 2 .. 4 parts that run side by side; one part owns the tile and
 * starts from (or, without a full wave before it, ends by adding) the other parts' exact s32 partial sums, which
 * travel through the workspace b200_int4_gemms_dense_workspace_bytes asks for: bit-identical results, no atomics on
 * data.  AUTO uses it for launches without a full wave whose parts keep at least 32 K blocks (few tiles, long
 * reductions: up to 1.4 x faster); ALWAYS also where full waves precede the tail (parts of at least 4 K blocks; at
 * 4096^3 the measured gain was within noise); OFF: whole tiles only.  Without a workspace whole tiles are scheduled. */
enum { B200_TAIL_AUTO = 0, B200_TAIL_OFF = 1, B200_TAIL_ALWAYS = 2 };

/* Tile width of per-channel int4 CTA-pair launches with a B stored [K, N] and bf16 output (dense, and grouped
 * forward).  A pair can own a 256 x 512 tile instead of 256 x 256: each CTA then unpacks its rows of A once per K
 * block for two blocks of B (a quarter less unpack work and shared-memory traffic per output element; one
 * accumulator fills TMEM, so the epilogue of a tile is not hidden behind the next tile).  AUTO takes wide tiles when
 * their waves, at 0.9 of the time of two narrow tiles each, need less time than the narrow tiles' waves; OFF / ON
 * force either (ON falls back where no wide kernel exists).  Where the wide tiles leave a thin last wave (at most
 * eight full waves before it, N a multiple of 512, tail_balance not OFF) three 512-column tiles of a row are traded
 * for four of 384 columns (second MMA with N = 128) until the last wave holds 384-column tiles only: at 4096^3, 74
 * tiles of 512 and 72 of 384 columns instead of 128 of 512, 52.1 -> 49.8 us.  Bit-identical results. */
enum { B200_WIDE_AUTO = 0, B200_WIDE_OFF = 1, B200_WIDE_ON = 2 };

typedef struct b200_gemm_variant {
  int32_t dtype;      /* B200_DTYPE_*      */
  int32_t layout;     /* B200_LAYOUT_*     */
  int32_t scale_mode; /* B200_SCALE_*      */
  int32_t subchannel; /* 32/64/128/256 when scale_mode is SUBCHANNEL, else 0 */
  int32_t epilogue;   /* B200_EPILOGUE_*   */
  int32_t out_dtype;  /* B200_OUT_*        */
  int32_t split_k;    /* 1, 2, 4 or 8 slices of K reduced by different CTAs and added by a second kernel in a
                         fixed order; >1 requires epilogue NONE, out_dtype F32 and a workspace */
  int32_t path;       /* B200_PATH_*       */
  int32_t group_m;    /* raster swizzle width in row tiles, 0 = library default */
  int32_t schedule;   /* B200_SCHEDULE_*   */
  int32_t cta_group;  /* B200_CTA_GROUP_*: SMs per output tile of the tensor-core kernel */
  int32_t accumulate_order; /* B200_ACCUMULATE_*: subchannel dense launches only */
  int32_t a_operand;  /* B200_A_OPERAND_* */
  int32_t tail_balance; /* B200_TAIL_* */
  int32_t task_align; /* grouped forward: what every task's block_start is a multiple of (the align_tile the tasks were
                         built with), as promised by the caller; 0 = not stated.  A transposed lhs (TN / TT) puts the
                         task's first row on the TMA x axis, which wants multiples of 16 bytes: the tensor-core path
                         takes it only with task_align a multiple of 16, otherwise the CUDA-core kernel runs.  A task
                         that breaks the promise is skipped and reported (code 4 of b200_int4_gemms_device_status) */
  int32_t wide_tiles; /* B200_WIDE_* */
} b200_gemm_variant;

/* Replaces amd_strix_halo_kernels_dispatch_version (dispatch.cpp:206). */
int b200_int4_gemms_dispatch_version(void);
/* Replaces amd_strix_halo_kernels_has_compiled_code_objects (dispatch.cpp:208): 1 when the
 * library was built with its sm_100a kernels. */
int b200_int4_gemms_has_compiled_kernels(void);
/* Replaces amd_strix_halo_kernels_has_hip_runtime (dispatch.cpp:212): 1 when a CUDA driver
 * and at least one device are usable from this process. */
int b200_int4_gemms_has_cuda_runtime(void);
/* Replaces amd_strix_halo_kernels_has_linked_kernels (dispatch.cpp:216): both of the above
 * and at least one visible device is compute capability 10.x. */
int b200_int4_gemms_has_linked_kernels(void);
/* Replaces amd_strix_halo_kernels_last_error (dispatch.cpp:220). */
const char* b200_int4_gemms_last_error(void);

/* Device-side status word of the most recent launches on a device: 0 = no kernel reported
 * a problem, 1 = a bounded wait inside a kernel ran out (the kernel gave up and returned),
 * 3 = a grouped forward launch was given a device-built task list that had overflowed its arrays,
 * 4 = a grouped forward launch with a transposed lhs met a task that does not start on a multiple of 16 rows although
 * variant->task_align promised it (detail[0] = the task, which was skipped).
 * Reading it does not synchronise; call it after synchronising the stream.  detail[0..2]
 * (may be NULL) receive the block index and wait site.  No reference counterpart. */
int b200_int4_gemms_device_status(int device_index, int32_t* detail);
/* Clears the status word. */
int b200_int4_gemms_reset_device_status(int device_index);

/* Dense GEMM:  C = epilogue((A_q @ B_q) * a_scale * b_scale).
 * Replaces amd_strix_halo_kernels_launch_hsaco (dispatch.cpp:224-283).
 *   a, b       operands in variant->layout (see above); for SWIGLU, B has 2*n output columns
 *              laid out [up | gate] and c has n columns.
 *   a_scale    bf16 [m] (per-channel) or [m, ceil(k/S)] (subchannel)
 *   b_scale    bf16 [cols] or [ceil(k/S), cols], cols = n (2*n for SWIGLU)
 *   c          [m, n] in variant->out_dtype
 *   workspace  device scratch (16-byte aligned) of b200_int4_gemms_dense_workspace_bytes(...) bytes: required
 *              for split_k > 1; optional otherwise (the balanced tail of B200_TAIL_AUTO is used only when it is
 *              there).  Launches that share a workspace must not overlap in time.  The first 4 KB hold flag words
 *              that must be zero before a launch and are left zero by it: the library clears them itself the first
 *              time it sees a workspace (address, size, device), so pass freshly allocated memory as it is; after
 *              freeing a workspace, or after a kernel reported a failed wait, call
 *              b200_int4_gemms_reset_device_status, which also makes the library clear the flag words again
 *   m, n, k    logical sizes (k counts int4 values, not bytes) */
int b200_int4_gemms_launch_dense(const b200_gemm_variant* variant, int device_index,
                                 uintptr_t stream_handle, const void* a, const void* b,
                                 const void* a_scale, const void* b_scale, void* c,
                                 void* workspace, size_t workspace_bytes, int32_t m, int32_t n,
                                 int32_t k);
size_t b200_int4_gemms_dense_workspace_bytes(const b200_gemm_variant* variant, int32_t m,
                                             int32_t n, int32_t k);

/* Split-K (variant->split_k = 2, 4, 8; the reference's SPLIT_K kernels, scripts/generate_amdgcn.py:189-192,
 * whose fp32 output the caller zero-fills, native.py:739-740).  Here K is cut into slices of whole 128-deep
 * K blocks (whole K-groups for subchannel scales); each slice is reduced by its own CTAs into the workspace
 * ([slices, m, n]; exact s32 partial sums for per-channel scales, fp32 partial sums for subchannel scales)
 * and a second kernel adds the slices in ascending order and, for per-channel scales, applies the scales
 * once.  No atomics: results are bit-identical from run to run, and for per-channel scales bit-identical
 * to split_k = 1.  The output needs no zero-fill.  Fewer slices than asked for are used when K is short. */

/* What b200_int4_gemms_launch_dense would do for a variant and shape on a device, without launching:
 * the kernel form, its grid and tile, the raster width and the effective split.  No reference counterpart
 * (the reference's caller computes the grid itself, native.py:306-332). */
enum {
  B200_LAUNCHED_NOTHING = 0,
  B200_LAUNCHED_TCGEN05 = 1,      /* tensor-core kernel, one CTA per tile */
  B200_LAUNCHED_TCGEN05_PAIR = 2, /* tensor-core kernel, CTA pair per tile */
  B200_LAUNCHED_SIMT = 3          /* CUDA-core kernel: correct, far slower; shapes and layouts the
                                     tensor-core kernel does not take */
};
typedef struct b200_dense_plan {
  int32_t path;      /* B200_LAUNCHED_* */
  int32_t grid;      /* CTAs */
  int32_t tile_rows; /* output rows per scheduled tile: 128, or 256 for a CTA pair */
  int32_t tile_cols; /* 256, or 128 for SwiGLU (up + gate) */
  int32_t group_m;   /* raster width in row tiles */
  int32_t split_k;   /* slices actually used */
  int32_t tail_units; /* > 0: the balanced tail is used, over this many CTAs (pairs), given a workspace */
  int32_t tiles_384; /* wide tiles only: tiles of 384 instead of 512 columns (mixed column cuts for a thin last wave) */
} b200_dense_plan;
int b200_int4_gemms_plan_dense(const b200_gemm_variant* variant, int device_index, int32_t m, int32_t n,
                               int32_t k, b200_dense_plan* plan);
/* B200_LAUNCHED_* of the most recent launch call made by the calling thread (dense or grouped):
 * lets a caller of B200_PATH_AUTO see that a launch went to the CUDA-core kernel. */
int b200_int4_gemms_last_launch_path(void);

/* Grouped forward (M-ragged):  out[rows of group g] = (lhs_rows @ rhs[g]) * a_scale * b_scale[g].
 * Replaces amd_strix_halo_kernels_launch_ragged_fwd_hsaco (dispatch.cpp:286-389).
 *   lhs        int4 [m, k_packed] (NN/NT) or [k_packed, m] (TN/TT)
 *   rhs        int4 [groups, k_packed, n] (NN/TN) or [groups, n, k_packed] (NT/TT)
 *   lhs_scale  bf16 [m] or [m, scale_cols];  rhs_scale bf16 [groups, n] or [groups, scale_cols, n]
 *   task_*     int64 [num_tasks] row-block tasks as built by calculate_group_info
 *              (reference ragged.py:201-323); block_rows = the tile they were built with (<= 256;
 *              tasks of more than 128 rows run on pairs of SMs and need per-channel scales or K-groups of
 *              at least 128 on the tensor-core path).  The tensor-core path takes a row-major lhs
 *              (layouts NN and NT) and, when variant->task_align is a multiple of 16 and m is one too, a
 *              transposed lhs (TN / TT, tasks of at most 128 rows); else TN / TT run on the CUDA-core kernel
 *   out        [m, n] bf16 or f32; rows outside every task's [actual_start, actual_end) are untouched */
int b200_int4_gemms_launch_ragged_fwd(const b200_gemm_variant* variant, int device_index,
                                      uintptr_t stream_handle, const void* lhs, const void* rhs,
                                      const void* lhs_scale, const void* rhs_scale,
                                      const int64_t* task_group_ids,
                                      const int64_t* task_block_starts,
                                      const int64_t* task_actual_starts,
                                      const int64_t* task_actual_ends, void* out, int32_t m,
                                      int32_t n, int32_t k_packed, int32_t scale_cols,
                                      int32_t num_tasks, int32_t groups, int32_t block_rows);

/* Grouped backward (K-ragged):  out[g] = (lhs[g][:, :k_g] @ rhs[g][:k_g, :]) * a_scale[g] * b_scale[g],
 * k_g = group_sizes[g]; entries beyond k_g (padding, and the odd tail nibble) are ignored;
 * an empty group produces zeros.
 * Replaces amd_strix_halo_kernels_launch_ragged_bwd_hsaco (dispatch.cpp:391-456).
 *   lhs        int4 [groups, m, k_packed] (NN/NT) or [groups, k_packed, m] (TN/TT)
 *   rhs        int4 [groups, k_packed, n] (NN/TN) or [groups, n, k_packed] (NT/TT)
 *   lhs_scale  bf16 [groups, m] or [groups, m, scale_cols]; rhs_scale [groups, n] or [groups, scale_cols, n]
 *   group_sizes int64 [groups]
 *   out        f32 [groups, m, n]
 * All four layouts run on the tensor cores (a K-major rhs with its bytes past k_g zeroed while it is unpacked).
 * Split-K is not needed for determinism here: every output tile is owned by one CTA, so
 * results are bit-identical from run to run. */
int b200_int4_gemms_launch_ragged_bwd(const b200_gemm_variant* variant, int device_index,
                                      uintptr_t stream_handle, const void* lhs, const void* rhs,
                                      const void* lhs_scale, const void* rhs_scale,
                                      const int64_t* group_sizes, void* out, int32_t m, int32_t n,
                                      int32_t k_packed, int32_t scale_cols, int32_t groups);

/* Expands packed int4 [rows, cols_packed] to int8 [rows, 2*cols_packed] (values -8..7,
 * even k from the low nibble).  The A/B comparison partner of the fused unpack path:
 * expand once, then run the int8 GEMM.  No reference counterpart (the reference only
 * unpacks on the host, quant.py:41-51). */
int b200_int4_gemms_unpack_int4(int device_index, uintptr_t stream_handle, const void* packed,
                                void* out_int8, int64_t rows, int64_t cols_packed);

/* ---- Callers and data formats either side of the GEMM path ------------------------------------ */

/* Row-block tasks of the grouped forward pass, built on the device: the CUDA counterpart of the
 * reference's task builder (ragged.py:127-185 Triton kernel, :201-323 calculate_group_info).
 * For group g with rows [s, e): aligned = floor(s / align) * align; task b of the group has
 * block_start = aligned + b * tile, actual_start = max(block_start, s), actual_end = min(block_start +
 * tile, e); empty groups make no task; tasks are written in group order.
 *   group_sizes   int64 [groups] on the device
 *   task_*        int64 [max_tasks] outputs; entries past the task count are empty tasks (all zero)
 *   num_tasks_dev int32 [1] output: min(task count, max_tasks)
 *   overflow_dev  int32 [1] output: 1 when the tasks did not fit in max_tasks (then the arrays hold the
 *                 first max_tasks tasks), else 0.  rows / tile + 2 * groups tasks always fit.
 * Nothing returns to the host: pair it with b200_int4_gemms_launch_ragged_fwd_device_tasks. */
int b200_int4_gemms_group_info(int device_index, uintptr_t stream_handle, const int64_t* group_sizes,
                               int32_t groups, int32_t tile, int32_t align, int64_t* task_group_ids,
                               int64_t* task_block_starts, int64_t* task_actual_starts,
                               int64_t* task_actual_ends, int32_t max_tasks, int32_t* num_tasks_dev,
                               int32_t* overflow_dev);

/* b200_int4_gemms_launch_ragged_fwd with the task count left on the device (num_tasks_dev, as written
 * by b200_int4_gemms_group_info); max_tasks is the capacity of the task arrays.  overflow_dev (may be
 * NULL) is the builder's overflow flag: when it is set the kernel still runs the tasks that fit, and
 * reports code 3 (detail[0] = tasks kept) through b200_int4_gemms_device_status, because rows of the
 * tasks that did not fit stay unwritten.  Task bounds are clamped to [0, m] on the device.  No reference
 * counterpart: the reference reads the task count back to the host (ragged.py:275). */
int b200_int4_gemms_launch_ragged_fwd_device_tasks(
    const b200_gemm_variant* variant, int device_index, uintptr_t stream_handle, const void* lhs,
    const void* rhs, const void* lhs_scale, const void* rhs_scale, const int64_t* task_group_ids,
    const int64_t* task_block_starts, const int64_t* task_actual_starts,
    const int64_t* task_actual_ends, const int32_t* num_tasks_dev, const int32_t* overflow_dev, void* out,
    int32_t m, int32_t n, int32_t k_packed, int32_t scale_cols, int32_t max_tasks, int32_t groups,
    int32_t block_rows);

/* Grouped backward over FLAT operands: all tokens back to back, no per-group padding.
 *   out[g] = (lhs[tokens of g, :]^T @ rhs[tokens of g, :]) * a_scale[g] * b_scale[g]
 * No reference counterpart: the reference API only takes operands stacked per group and padded to a
 * common capacity (ragged.py:1232-1402); this entry removes that repack.
 *   variant     int4, layout TN, per-channel scales, no epilogue, f32 output
 *   lhs         int4 [ceil(tokens/2), m]: byte (p, i) holds tokens 2p (low nibble) and 2p+1 of feature i
 *   rhs         int4 [ceil(tokens/2), n], same packing (b200_int4_gemms_repack_tokens makes both)
 *   lhs_scale   bf16 [groups, m]; rhs_scale bf16 [groups, n]
 *   group_sizes int64 [groups], summing to tokens; groups may start on odd tokens
 *   out         f32 [groups, m, n]
 *   workspace   device scratch, 8-byte aligned, b200_int4_gemms_ragged_bwd_flat_workspace_bytes(groups)
 *               bytes: the first token of every group, written by a small scan kernel launched first
 *               on the same stream.  Calls that share a workspace must not overlap.
 * A single group must stay below 131072 tokens (accumulator headroom of the int4 encoding). */
size_t b200_int4_gemms_ragged_bwd_flat_workspace_bytes(int32_t groups);
int b200_int4_gemms_launch_ragged_bwd_flat(const b200_gemm_variant* variant, int device_index,
                                           uintptr_t stream_handle, const void* lhs, const void* rhs,
                                           const void* lhs_scale, const void* rhs_scale,
                                           const int64_t* group_sizes, void* out, void* workspace,
                                           size_t workspace_bytes, int32_t m, int32_t n, int64_t tokens,
                                           int32_t groups);

/* b200_int4_gemms_launch_ragged_bwd_flat for callers that can neither hand over device scratch nor
 * let the library allocate: code running inside someone else's memory plan (a framework whose pool
 * is fully reserved, a plugin that is told not to touch the allocator because allocation would
 * synchronise the device or move what the host application has placed).  No reference counterpart.
 * Same arguments minus the workspace.  The group starts go to an array that is part of the library
 * image (B200_STATIC_SCRATCH_MAX_GROUPS + 1 int64 entries, 32 KB + 8 bytes per device); nothing is
 * allocated on any call, the first included.
 *   - more than B200_STATIC_SCRATCH_MAX_GROUPS groups: refused (rc 1, message names the limit);
 *   - the first call on a device also looks the array's address up and sets the GEMM kernel's
 *     shared-memory attribute: make one call before starting a stream capture, since that set-up
 *     is host-side work that does not belong inside one;
 *   - the array is shared by all calls on a device and keeps what the last call wrote.  Each call
 *     rewrites the entries it reads, so nothing needs clearing, but two calls that can overlap in
 *     time (two streams, two threads) race on it: serialise them, or use the workspace form;
 *   - a bounded device wait that runs out is reported through b200_int4_gemms_device_status only
 *     when another entry point has already set the device up (that set-up owns the status word). */
#define B200_STATIC_SCRATCH_MAX_GROUPS 4096
int b200_int4_gemms_launch_ragged_bwd_flat_static(const b200_gemm_variant* variant, int device_index,
                                                  uintptr_t stream_handle, const void* lhs,
                                                  const void* rhs, const void* lhs_scale,
                                                  const void* rhs_scale, const int64_t* group_sizes,
                                                  void* out, int32_t m, int32_t n, int64_t tokens,
                                                  int32_t groups);

/* bf16 [rows, cols] -> quantisation codes clamp(round_half_even(float(x) / scale), qmin, qmax):
 * bits = 4: packed two per byte along the last axis (even index in the low nibble, an odd cols pads
 * with a zero code), dst u8 [rows, ceil(cols/2)]; bits = 8: dst int8 [rows, cols].
 * GPU form of fake_quant_int followed by pack_int4_k_major (quant.py:14-38), bit-identical to them. */
int b200_int4_gemms_quantize(int device_index, uintptr_t stream_handle, const void* src_bf16, void* dst,
                             int64_t rows, int64_t cols, int32_t bits, float scale);

/* int4 packed along features, src u8 [rows, cols/2] (the forward operand format) -> packed along
 * tokens, dst u8 [ceil(rows/2), cols] (the flat backward operand format); cols even.  No reference
 * counterpart (the reference repacks on the host, tests/test_ragged_dot.py:55-81). */
int b200_int4_gemms_repack_tokens(int device_index, uintptr_t stream_handle, const void* src, void* dst,
                                  int64_t rows, int64_t cols);

#ifdef __cplusplus
}
#endif

#endif /* B200_INT4_GEMMS_H_ */
