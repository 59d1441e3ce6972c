// C ABI of libb200_int4_gemms.so (declared in include/b200_int4_gemms.h): argument checks,
// TMA tensor-map construction, kernel selection and launch.  Plays the part of the
// reference's native/src/dispatch.cpp, with the kernels linked in.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/b200_int4_gemms.h"
#include <vector>

#include "tc_table.h"
#include "simt_kernel.cuh"
#include "prep_kernels.cuh"

namespace {

using namespace b200;

thread_local std::string g_last_error;

int fail(std::string msg) {
  g_last_error = std::move(msg);
  return 1;
}

int fail_cuda(const char* what, cudaError_t err) {
  // clear the (non-sticky) error so that the next call starts clean
  (void)cudaGetLastError();
  return fail(std::string(what) + " failed: " + cudaGetErrorString(err));
}

// ---------------------------------------------------------------------------------------
// driver entry point for tensor maps (no link-time dependency on libcuda)
// ---------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_init_mutex;
EncodeTiledFn g_encode_tiled = nullptr;
bool g_encode_attempted = false;

EncodeTiledFn encode_tiled_fn() {
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (g_encode_attempted) return g_encode_tiled;
  g_encode_attempted = true;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess && fn != nullptr) {
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  } else {
    (void)cudaGetLastError();
  }
  return g_encode_tiled;
}

// 2-D byte tensor map: inner extent `inner_bytes` (pitch `pitch_bytes`), `rows` rows.
int make_map_2d(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows,
                uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, int swizzle_bytes,
                const char* name) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail("cuTensorMapEncodeTiled is not available from this CUDA driver");
  const cuuint64_t dims[2] = {inner_bytes, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                  elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                       : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(std::string("cuTensorMapEncodeTiled failed for ") + name + " (CUresult " +
                std::to_string(static_cast<int>(r)) + ")");
  }
  return 0;
}

// ---------------------------------------------------------------------------------------
// per-device state: SM count, host-mapped status word, one-time kernel attribute set-up
// ---------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  int max_pair_clusters = 0;  // clusters of two CTAs the device can hold at once (pair kernels)
  int* status_host = nullptr;  // pinned + mapped
  int* status_dev = nullptr;
};
DeviceState g_devices[kMaxDevices];
std::mutex g_device_mutex;

// ---------------------------------------------------------------------------------------
// the tensor-core kernels this library holds (compiled in tc_kernels.cu, several parts)
// ---------------------------------------------------------------------------------------
const std::vector<TcKernelInfo>& tc_kernels() {
  static const std::vector<TcKernelInfo> table = [] {
    std::vector<TcKernelInfo> t;
    tc_register_part_0(t);
    tc_register_part_1(t);
    tc_register_part_2(t);
    tc_register_part_3(t);
    tc_register_part_4(t);
    tc_register_part_5(t);
    tc_register_part_6(t);
    tc_register_part_7(t);
    return t;
  }();
  return table;
}

struct TcLaunch {
  bool int4, a_mn, b_mn, mask_k;
  int scale, epi, out;
  bool pair = false;     // CTA-pair kernel (clusters of two, 256-row tiles)
  int flavor = FLAVOR_PLAIN;  // FLAVOR_FUSED_SC: fused subchannel order; FLAVOR_TMEM_A: A operand through TMEM
};

const TcKernelInfo* tc_find(const TcLaunch& l) {
  for (const TcKernelInfo& k : tc_kernels()) {
    if (k.int4 == l.int4 && k.a_mn == l.a_mn && k.b_mn == l.b_mn && k.scale == l.scale && k.epi == l.epi &&
        k.out == l.out && k.mask_k == l.mask_k && k.pair == l.pair && k.flavor == l.flavor)
      return &k;
  }
  return nullptr;
}

bool tc_has(const TcLaunch& l) { return tc_find(l) != nullptr; }

// One-time set-up of one kernel on the current device: its dynamic shared-memory size and, for kernels that
// re-balance registers between roles with setmaxnreg, a check of the compiled register count.  setmaxnreg.inc
// waits for ever if the CTA's register pool is smaller than the roles ask for, .inc may not lower and .dec may
// not raise a warp's count: a build whose compiler allocated differently is refused here, with a message,
// instead of faulting or hanging on the device.  Allocates nothing.
int prepare_kernel(const TcKernelInfo& k) {
  cudaError_t err = cudaFuncSetAttribute(k.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k.smem_bytes);
  if (err != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(max dynamic shared memory)", err);
  if (k.reg_pool_needed > 0) {
    cudaFuncAttributes attr;
    err = cudaFuncGetAttributes(&attr, k.fn);
    if (err != cudaSuccess) return fail_cuda("cudaFuncGetAttributes", err);
    const bool pool_ok = attr.numRegs * k.threads >= k.reg_pool_needed;
    const bool moves_ok = attr.numRegs >= k.regs_light && attr.numRegs <= k.regs_epilogue &&
                          (k.unpack_warps == 0 ||
                           (k.unpack_raises ? attr.numRegs <= k.regs_unpack : attr.numRegs >= k.regs_unpack));
    if (!pool_ok || !moves_ok)
      return fail("a kernel was compiled with " + std::to_string(attr.numRegs) +
                  " registers per thread, which does not fit its setmaxnreg register re-balance");
  }
  return 0;
}

void cluster_launch_config(const TcKernelInfo& k, int grid, cudaStream_t stream, cudaLaunchConfig_t* cfg,
                           cudaLaunchAttribute* attr) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(grid);
  cfg->blockDim = dim3(k.threads);
  cfg->dynamicSmemBytes = k.smem_bytes;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = k.pair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

int ensure_device(int device_index, DeviceState** out) {
  if (device_index < 0 || device_index >= kMaxDevices) return fail("device_index out of range");
  cudaError_t err = cudaSetDevice(device_index);
  if (err != cudaSuccess) return fail_cuda("cudaSetDevice", err);
  std::lock_guard<std::mutex> lock(g_device_mutex);
  DeviceState& st = g_devices[device_index];
  if (!st.ready) {
    cudaDeviceProp prop;
    err = cudaGetDeviceProperties(&prop, device_index);
    if (err != cudaSuccess) return fail_cuda("cudaGetDeviceProperties", err);
    st.sm_count = prop.multiProcessorCount;
    st.cc_major = prop.major;
    if (prop.major != 10) {
      return fail("this library holds sm_100a kernels only; device " + std::to_string(device_index) +
                  " is compute capability " + std::to_string(prop.major) + "." +
                  std::to_string(prop.minor));
    }
    err = cudaHostAlloc(reinterpret_cast<void**>(&st.status_host), 4 * sizeof(int), cudaHostAllocMapped);
    if (err != cudaSuccess) return fail_cuda("cudaHostAlloc(status)", err);
    std::memset(st.status_host, 0, 4 * sizeof(int));
    err = cudaHostGetDevicePointer(reinterpret_cast<void**>(&st.status_dev), st.status_host, 0);
    if (err != cudaSuccess) return fail_cuda("cudaHostGetDevicePointer(status)", err);
    // CTA-pair kernels are persistent: every cluster of the grid must be resident at once, so the grid
    // is sized by what the device can co-schedule (not every SM can always be paired).
    st.max_pair_clusters = st.sm_count / 2;
    for (const TcKernelInfo& k : tc_kernels()) {
      if (int rc = prepare_kernel(k); rc != 0) return rc;
      if (!k.pair) continue;
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute attr[1];
      cluster_launch_config(k, st.sm_count & ~1, nullptr, &cfg, attr);
      int clusters = 0;
      err = cudaOccupancyMaxActiveClusters(&clusters, k.fn, &cfg);
      if (err != cudaSuccess) return fail_cuda("cudaOccupancyMaxActiveClusters", err);
      if (clusters < st.max_pair_clusters) st.max_pair_clusters = clusters;
    }
    st.ready = true;
  }
  *out = &st;
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Output map for the TMA-store epilogue: [rows, n] elements of 2 (bf16) or 4 (f32) bytes, box of
// 32 rows x 32 columns (64 or 128 bytes, swizzle of the same width).  Returns 1 in *enabled when the output qualifies.
int make_output_map(CUtensorMap* map, void* out, int out_dtype, uint64_t rows, uint64_t n, int* enabled) {
  *enabled = 0;
  std::memset(map, 0, sizeof(*map));
  if (out_dtype == OUT_S32) return 0;
  const uint64_t esize = out_dtype == OUT_F32 ? 4 : 2;
  if (!aligned16(out) || (n * esize) % 16 != 0) return 0;
  // bf16: 32 columns = 64 bytes per row; f32: 32 columns = 128 bytes per row
  const uint32_t inner = out_dtype == OUT_F32 ? 128 : 64;
  if (int rc = make_map_2d(map, out, n * esize, rows, n * esize, inner, 32, static_cast<int>(inner), "C"); rc != 0) return rc;
  *enabled = 1;
  return 0;
}

int launch_tc(const TcLaunch& l, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
              const GemmParams& p, int grid, cudaStream_t stream) {
  const TcKernelInfo* k = tc_find(l);
  if (k == nullptr) return -1;  // no such instantiation
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  cluster_launch_config(*k, grid, stream, &cfg, attr);
  void* args[4] = {const_cast<CUtensorMap*>(&ta), const_cast<CUtensorMap*>(&tb), const_cast<CUtensorMap*>(&tc),
                   const_cast<GemmParams*>(&p)};
  cudaError_t err = cudaLaunchKernelExC(&cfg, k->fn, args);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("tcgen05 GEMM kernel launch", err);
  return 0;
}

int check_variant(const b200_gemm_variant* v) {
  if (v == nullptr) return fail("variant must be non-null");
  if (v->dtype != B200_DTYPE_INT4 && v->dtype != B200_DTYPE_INT8) return fail("variant.dtype is not INT4 or INT8");
  if (v->layout < B200_LAYOUT_NN || v->layout > B200_LAYOUT_TT) return fail("variant.layout is not NN, NT, TN or TT");
  if (v->scale_mode == B200_SCALE_SUBCHANNEL) {
    if (v->subchannel != 32 && v->subchannel != 64 && v->subchannel != 128 && v->subchannel != 256)
      return fail("variant.subchannel must be 32, 64, 128 or 256");
  } else if (v->scale_mode != B200_SCALE_PER_CHANNEL) {
    return fail("variant.scale_mode is not PER_CHANNEL or SUBCHANNEL");
  }
  if (v->epilogue < B200_EPILOGUE_NONE || v->epilogue > B200_EPILOGUE_SWIGLU) return fail("variant.epilogue is unknown");
  if (v->out_dtype < B200_OUT_BF16 || v->out_dtype > B200_OUT_S32) return fail("variant.out_dtype is unknown");
  if (v->out_dtype == B200_OUT_S32 && (v->scale_mode != B200_SCALE_PER_CHANNEL || v->epilogue != B200_EPILOGUE_NONE))
    return fail("out_dtype S32 (raw accumulators) needs per-channel mode and no epilogue");
  if (v->split_k != 1 && v->split_k != 2 && v->split_k != 4 && v->split_k != 8) return fail("variant.split_k must be 1, 2, 4 or 8");
  if (v->split_k > 1 && (v->epilogue != B200_EPILOGUE_NONE || v->out_dtype != B200_OUT_F32))
    return fail("split_k > 1 needs epilogue NONE and float32 output");
  if (v->path < B200_PATH_AUTO || v->path > B200_PATH_SIMT) return fail("variant.path is unknown");
  if (v->schedule != B200_SCHEDULE_PERSISTENT && v->schedule != B200_SCHEDULE_TILE_PER_CTA)
    return fail("variant.schedule is unknown");
  if (v->cta_group < B200_CTA_GROUP_AUTO || v->cta_group > B200_CTA_GROUP_PAIR) return fail("variant.cta_group is unknown");
  if (v->accumulate_order != B200_ACCUMULATE_FUSED && v->accumulate_order != B200_ACCUMULATE_REFERENCE)
    return fail("variant.accumulate_order is unknown");
  if (v->a_operand < B200_A_OPERAND_AUTO || v->a_operand > B200_A_OPERAND_TMEM) return fail("variant.a_operand is unknown");
  if (v->tail_balance < B200_TAIL_AUTO || v->tail_balance > B200_TAIL_ALWAYS) return fail("variant.tail_balance is unknown");
  if (v->wide_tiles < B200_WIDE_AUTO || v->wide_tiles > B200_WIDE_ON) return fail("variant.wide_tiles is unknown");
  return 0;
}

int launch_simt(const SimtParams& sp, int rows_per_z, int z, cudaStream_t stream) {
  if (sp.N <= 0 || rows_per_z <= 0 || z <= 0) return 0;
  dim3 grid((sp.N + 63) / 64, (rows_per_z + 3) / 4, z);
  if (grid.y > 65535 || grid.z > 65535) return fail("problem too large for the CUDA-core kernel's grid");
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(sp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("CUDA-core GEMM kernel launch", err);
  return 0;
}

// The flag words of a balanced-tail workspace must be zero before its first launch; the kernels leave them zero.  The
// library clears them when it first sees a workspace (address, size, device) and remembers the last few it has seen,
// so that back-to-back launches do not carry a memset between them.
struct SeenWorkspace {
  const void* ptr = nullptr;
  size_t bytes = 0;
  int device = -1;
};
constexpr int kSeenWorkspaces = 32;
SeenWorkspace g_seen_workspaces[kSeenWorkspaces];
int g_seen_next = 0;
std::mutex g_seen_mutex;

void forget_workspaces(int device) {
  std::lock_guard<std::mutex> lock(g_seen_mutex);
  for (SeenWorkspace& w : g_seen_workspaces)
    if (w.device == device) w = SeenWorkspace{};
}

bool workspace_seen_before(const void* ptr, size_t bytes, int device) {
  std::lock_guard<std::mutex> lock(g_seen_mutex);
  for (const SeenWorkspace& w : g_seen_workspaces)
    if (w.ptr == ptr && w.bytes == bytes && w.device == device) return true;
  g_seen_workspaces[g_seen_next] = SeenWorkspace{ptr, bytes, device};
  g_seen_next = (g_seen_next + 1) % kSeenWorkspaces;
  return false;
}
}  // namespace

extern "C" int b200_int4_gemms_dispatch_version(void) { return 1; }

extern "C" int b200_int4_gemms_has_compiled_kernels(void) { return 1; }

extern "C" int b200_int4_gemms_has_cuda_runtime(void) {
  int count = 0;
  cudaError_t err = cudaGetDeviceCount(&count);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return count > 0 ? 1 : 0;
}

extern "C" int b200_int4_gemms_has_linked_kernels(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  for (int device = 0; device < count; ++device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
      (void)cudaGetLastError();
      continue;
    }
    if (major == 10) return 1;
  }
  return 0;
}

extern "C" const char* b200_int4_gemms_last_error(void) { return g_last_error.c_str(); }

extern "C" int b200_int4_gemms_device_status(int device_index, int32_t* detail) {
  if (device_index < 0 || device_index >= kMaxDevices) return 0;
  DeviceState& st = g_devices[device_index];
  if (!st.ready || st.status_host == nullptr) return 0;
  volatile int* s = st.status_host;
  if (detail != nullptr) {
    detail[0] = s[1];
    detail[1] = s[2];
    detail[2] = s[3];
  }
  return s[0];
}

extern "C" int b200_int4_gemms_reset_device_status(int device_index) {
  if (device_index < 0 || device_index >= kMaxDevices) return 1;
  forget_workspaces(device_index);  // a kernel that gave up may have left flag words set: clear them at the next launch
  DeviceState& st = g_devices[device_index];
  if (st.ready && st.status_host != nullptr) std::memset(st.status_host, 0, 4 * sizeof(int));
  return 0;
}

namespace {

// Everything launch_dense decides before it launches: the kernel form, the tile grid, the split.
struct DensePlan {
  bool tensor_core = false;
  TcLaunch kernel{};
  int tile_rows = BM;
  int tile_cols = BN;
  int tiles_m = 0, tiles_n = 0;
  int group_m = 1;
  int grid = 0;
  int slices = 1;        // effective split-K factor (<= variant.split_k)
  int k_per_slice = 0;
  bool integer_partials = false;
  int tail_units = 0;    // > 0: balanced tail over this many scheduling units (needs the workspace)
  int tail_split = 0, tail_waves = 0, tail_rest = 0;
  // wide kernel, mixed column cuts (GemmParams::mix_*); mix_total_wide < 0: all tiles 512 columns wide
  int mix_total_wide = -1, mix_rows_hi = 0, mix_wide_hi = 0, mix_wide_lo = 0, mix_tq_hi = 0, mix_tq_lo = 0;
};

// Workspace of the balanced tail: one partial-sum slot of 2 x 128 x 256 s32 per scheduling unit, then the flags.
constexpr size_t kTailSlotBytes = 2u * BM * BN * sizeof(int);
// Layout: the flag words first (a fixed 4 KB, enough for kTailMaxUnits units, so that they sit in the same place
// whatever kernel form uses the workspace next), then one partial-sum slot per unit.
constexpr size_t kTailFlagBytes = 4096;
size_t tail_workspace_bytes(int units) { return kTailFlagBytes + static_cast<size_t>(units) * kTailSlotBytes; }

constexpr int kTailMaxUnits = 160;  // an upper bound on the SMs of a device, for sizing a workspace without one
static_assert(kTailMaxUnits * 4 * sizeof(int) <= 4096, "flag words of every unit fit the fixed flag area");

int effective_slices(int k, int unit, int requested, int* k_per_slice) {
  const int units = (k + unit - 1) / unit;
  const int want = requested < units ? requested : units;
  const int per = (units + want - 1) / want;  // units per slice
  *k_per_slice = per * unit;
  return (units + per - 1) / per;
}

// `a`, `b`, `c` only decide alignment; nullptr means "assume aligned".
int plan_dense(const b200_gemm_variant* v, const DeviceState* dev, const void* a, const void* b, int32_t m,
               int32_t n, int32_t k, size_t have_workspace_bytes, DensePlan* plan) {
  const bool int4 = v->dtype == B200_DTYPE_INT4;
  const bool swiglu = v->epilogue == B200_EPILOGUE_SWIGLU;
  const int b_cols = swiglu ? 2 * n : n;
  const int kb = int4 ? (k + 1) / 2 : k;
  const bool a_t = (v->layout == B200_LAYOUT_TN || v->layout == B200_LAYOUT_TT);
  const bool b_t = (v->layout == B200_LAYOUT_NT || v->layout == B200_LAYOUT_TT);
  const int sc_mode = (v->scale_mode == B200_SCALE_SUBCHANNEL) ? SCALE_SC : SCALE_PC;
  DensePlan pl;
  pl.tile_cols = swiglu ? NBLK : BN;
  pl.tiles_n = (n + pl.tile_cols - 1) / pl.tile_cols;

  // split-K: slices of whole K blocks (and whole K-groups); per-channel slices store exact s32 partial sums,
  // subchannel slices fp32 partial sums, and splitk_reduce_kernel adds them in slice order
  int out_kind = v->out_dtype;
  if (v->split_k > 1) {
    const int unit = (sc_mode == SCALE_SC && v->subchannel > BK) ? v->subchannel : BK;
    pl.slices = effective_slices(k, unit, v->split_k, &pl.k_per_slice);
    if (pl.slices > 1) {
      pl.integer_partials = sc_mode == SCALE_PC;
      out_kind = pl.integer_partials ? OUT_S32 : OUT_F32;
    }
  }
  TcLaunch tl{int4, a_t, !b_t, false, sc_mode, v->epilogue, out_kind};
  // subchannel scales: the fused accumulation order unless the caller asks for the reference's order of
  // roundings (or the variant has no kernel in the fused order, e.g. K-groups of 32 / 64 would gain nothing)
  if (sc_mode == SCALE_SC && v->accumulate_order == B200_ACCUMULATE_FUSED) {
    TcLaunch fused = tl;
    fused.flavor = FLAVOR_FUSED_SC;
    if (tc_has(fused)) tl = fused;
  }
  bool tc_ok = tc_has(tl) && (a == nullptr || aligned16(a)) && (b == nullptr || aligned16(b));
  tc_ok = tc_ok && ((a_t ? m : kb) % 16 == 0) && ((b_t ? kb : b_cols) % 16 == 0);  // TMA needs 16-byte pitches
  // fused SwiGLU reads the gate block at column n of a B stored [Kb, 2n]: a TMA x coordinate, multiples of 16 bytes
  if (swiglu && !b_t && n % 16 != 0) tc_ok = false;
  if (v->path == B200_PATH_SIMT) tc_ok = false;
  if (v->path == B200_PATH_TCGEN05 && !tc_ok)
    return fail("the tcgen05 kernel needs 16-byte aligned operands, operand pitches that are multiples of 16 bytes (for a fused SwiGLU over B [Kb, 2n]: n a multiple of 16), and a kernel instantiated for the variant");
  if (!tc_ok && pl.slices > 1)
    return fail("split_k > 1 runs on the tensor-core kernel only (layouts NN / NT per-channel, NN subchannel; 16-byte aligned operands and pitches)");
  pl.tensor_core = tc_ok;
  if (tc_ok) {
    // CTA pairs: 256-row tiles over two SMs.  A pair's K block takes about 0.87 of the time a single CTA needs
    // for its 128 x 256 tile (a third less operand traffic per SM), so pairs win whenever they do not need
    // more waves than that: compare waves x time per tile of the two schedules.  An M that is not a multiple
    // of 256 leaves the peer CTA of the last row of tiles without rows, which the wave count accounts for.
    TcLaunch pair = tl;
    pair.pair = true;
    const bool sc_ok = sc_mode == SCALE_PC || v->subchannel >= BK;
    const long long single_tiles = static_cast<long long>((m + BM - 1) / BM) * pl.tiles_n * pl.slices;
    const long long pair_tiles = static_cast<long long>((m + 2 * BM - 1) / (2 * BM)) * pl.tiles_n * pl.slices;
    const long long single_waves = (single_tiles + dev->sm_count - 1) / dev->sm_count;
    const int pairs = dev->max_pair_clusters > 0 ? dev->max_pair_clusters : 1;
    const long long pair_waves = (pair_tiles + pairs - 1) / pairs;
    const bool want = v->cta_group == B200_CTA_GROUP_PAIR ||
                      (v->cta_group == B200_CTA_GROUP_AUTO && m > BM && 87 * pair_waves <= 100 * single_waves);
    if (want && sc_ok && dev->max_pair_clusters > 0 && tc_has(pair)) tl = pair;
    pl.kernel = tl;
    pl.tile_rows = tl.pair ? 2 * BM : BM;
    pl.tiles_m = (m + pl.tile_rows - 1) / pl.tile_rows;
    // raster width (row tiles walked before the next column tile), from sweeps on a B200: 16 for the 256-row
    // tiles of CTA pairs, 32 for single-CTA int8 tiles, 8 for single-CTA int4 tiles
    pl.group_m = v->group_m > 0 ? v->group_m : (tl.pair ? 16 : (int4 ? 8 : 32));
    const int num_tiles = pl.tiles_m * pl.tiles_n * pl.slices;
    const int cta_per_tile = tl.pair ? 2 : 1;
    const int max_units = tl.pair ? dev->max_pair_clusters : dev->sm_count;  // tiles in flight
    pl.grid = (num_tiles < max_units ? num_tiles : max_units) * cta_per_tile;
    if (v->schedule == B200_SCHEDULE_TILE_PER_CTA) pl.grid = num_tiles * cta_per_tile;
    // Balanced tail: the tiles of a last wave that fills at most half of the units are cut along K into 2 .. 4 parts
    // that run side by side (per-channel scales: the partial sums that cross units are exact integers, so the result
    // does not change).  Worth it while one wave is a visible share of the run; needs the caller's workspace.
    const int kb_per_tile = (k + BK - 1) / BK;
    const int rest = num_tiles % max_units, waves = num_tiles / max_units;
    // AUTO keeps to launches without a full wave (few tiles, long reductions), where the gain is large; with full
    // waves before the tail the measured gain at 4096^3 was within noise for CTA pairs, so that takes ALWAYS.
    const bool tail_wanted = v->tail_balance == B200_TAIL_ALWAYS || (v->tail_balance == B200_TAIL_AUTO && waves == 0);
    if (tail_wanted && v->schedule == B200_SCHEDULE_PERSISTENT && sc_mode == SCALE_PC && pl.slices == 1 &&
        rest > 0 && waves <= 4 && have_workspace_bytes >= tail_workspace_bytes(max_units)) {
      // With a full wave before it the owner part starts from the other parts' sum, loaded while earlier tiles run:
      // parts of at least 4 K blocks pay.  Without one (fewer tiles than units) the parts run side by side and the
      // sums are added after the MMAs, a few serial trips to L2: only long reductions (32 K blocks per part) pay.
      const int min_part = waves > 0 ? 4 : 32;
      int split = max_units / rest;
      if (split > 4) split = 4;
      while (split >= 2 && kb_per_tile / split < min_part) --split;
      TcLaunch with_tail = tl;
      with_tail.flavor = FLAVOR_TAIL;
      if (split >= 2 && tl.flavor == FLAVOR_PLAIN && tc_has(with_tail)) {
        tl = with_tail;
        pl.kernel = tl;
        pl.tail_units = waves > 0 ? max_units : split * rest;  // no full wave: only the units that hold a part
        pl.tail_split = split;
        pl.tail_waves = waves;
        pl.tail_rest = rest;
        pl.grid = pl.tail_units * cta_per_tile;
      }
    }
    // per-channel int4 pairs with a row-major A: the kernel that keeps the unpacked A operand in TMEM
    // (one accumulator buffer: the epilogue of a tile is not hidden behind the next tile's MMAs, which the saved
    // shared-memory traffic outweighs from about 48 K blocks per tile on: +9 % at K = 8192, even at K = 4096)
    if (pl.tail_units == 0 && tl.pair && (v->a_operand == B200_A_OPERAND_TMEM || (v->a_operand == B200_A_OPERAND_AUTO && k >= 48 * BK))) {
      TcLaunch through_tmem = tl;
      through_tmem.flavor = FLAVOR_TMEM_A;
      if (tc_has(through_tmem)) tl = through_tmem;
    }
    // Wide tiles (256 x 512 per pair) where such a kernel exists: a wide tile takes 0.9 of the time of the two
    // narrow tiles it replaces (measured at 4096^3 and 8192^3), so they win when their waves need less time.
    // They come before A-through-TMEM (3650 against 3312 TOPS at 8192^3) and after the balanced tail, which AUTO
    // only takes for launches without a full wave.
    if (tl.pair && (tl.flavor == FLAVOR_PLAIN || tl.flavor == FLAVOR_TMEM_A) && pl.slices == 1 && pl.tail_units == 0 &&
        pl.tile_cols == BN && v->wide_tiles != B200_WIDE_OFF && v->schedule == B200_SCHEDULE_PERSISTENT) {
      TcLaunch wide = tl;
      wide.flavor = FLAVOR_WIDE;
      const int wide_cols = (n + 2 * BN - 1) / (2 * BN);
      const long long wide_waves = (static_cast<long long>(pl.tiles_m) * wide_cols + max_units - 1) / max_units;
      const long long narrow_waves = (static_cast<long long>(num_tiles) + max_units - 1) / max_units;
      if (tc_has(wide) && (v->wide_tiles == B200_WIDE_ON || 18 * wide_waves < 10 * narrow_waves)) {
        tl = wide;
        pl.tile_cols = 2 * BN;
        pl.tiles_n = wide_cols;
        const int wide_tiles = pl.tiles_m * pl.tiles_n;
        pl.grid = (wide_tiles < max_units ? wide_tiles : max_units) * cta_per_tile;
        if (v->group_m <= 0) pl.group_m = 4;  // with TMA four K blocks ahead the raster hardly matters; 1 .. 8 measured alike
        // A thin last wave: trade three 512-column tiles of a row for four of 384 columns (a 384-column tile takes
        // 0.9 of the time of a whole one) until the last wave holds 384-column tiles only.  Only where one wave is a
        // visible share of the run and N is whole 512-column tiles.
        const int rest_w = wide_tiles % max_units, full_w = wide_tiles / max_units;
        if (v->tail_balance != B200_TAIL_OFF && rest_w > 0 && full_w >= 1 && full_w <= 8 && n % (2 * BN) == 0) {
          const int swaps = (rest_w + 2) / 3;                       // each swap removes three wide tiles, adds four narrower
          const int spill = 3 * swaps - rest_w;                     // 384-column tiles that land in the last full wave
          const int per_row_max = wide_cols / 3;
          if (4 * swaps - spill <= max_units && swaps <= pl.tiles_m * per_row_max) {
            const int lo = swaps / pl.tiles_m, hi_rows = swaps % pl.tiles_m;   // swaps per row tile: lo, or lo + 1 for the first hi_rows
            pl.mix_rows_hi = hi_rows;
            pl.mix_wide_hi = wide_cols - 3 * (lo + 1);
            pl.mix_wide_lo = wide_cols - 3 * lo;
            pl.mix_tq_hi = 4 * (lo + 1);
            pl.mix_tq_lo = 4 * lo;
            pl.mix_total_wide = wide_tiles - 3 * swaps;
          }
        }
      }
    }
    pl.kernel = tl;
  } else {
    pl.tiles_m = (m + 3) / 4;  // the CUDA-core kernel: 4 rows x 64 columns per block
    pl.tiles_n = (n + 63) / 64;
    pl.grid = pl.tiles_m * pl.tiles_n;
  }
  *plan = pl;
  return 0;
}

thread_local int g_last_path = B200_LAUNCHED_NOTHING;

}  // namespace

extern "C" int b200_int4_gemms_last_launch_path(void) { return g_last_path; }

extern "C" size_t b200_int4_gemms_dense_workspace_bytes(const b200_gemm_variant* variant, int32_t m,
                                                        int32_t n, int32_t k) {
  if (variant == nullptr || m <= 0 || n <= 0 || k <= 0) return 0;
  if (variant->split_k <= 1) {
    // what the balanced tail would use if the launch qualifies for it (optional: without it whole tiles are scheduled)
    const long long tiles = static_cast<long long>((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const bool base = variant->scale_mode == B200_SCALE_PER_CHANNEL && variant->schedule == B200_SCHEDULE_PERSISTENT &&
                      variant->path != B200_PATH_SIMT;
    const bool may_balance = base && ((variant->tail_balance == B200_TAIL_ALWAYS && k >= 8 * BK) ||
                                      (variant->tail_balance == B200_TAIL_AUTO && tiles < kTailMaxUnits && k >= 64 * BK));
    return may_balance ? tail_workspace_bytes(kTailMaxUnits) : 0;
  }
  const int sc = variant->scale_mode == B200_SCALE_SUBCHANNEL ? variant->subchannel : 0;
  int per = 0;
  const int slices = effective_slices(k, sc > BK ? sc : BK, variant->split_k, &per);
  if (slices <= 1) return 0;
  return static_cast<size_t>(slices) * static_cast<size_t>(m) * static_cast<size_t>(n) * 4u;  // s32 or f32 partials
}

extern "C" int b200_int4_gemms_plan_dense(const b200_gemm_variant* v, int device_index, int32_t m, int32_t n,
                                          int32_t k, b200_dense_plan* out) {
  g_last_error.clear();
  if (int rc = check_variant(v); rc != 0) return rc;
  if (out == nullptr) return fail("plan must be non-null");
  if (m <= 0 || n <= 0 || k <= 0) return fail("m, n and k must be positive");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  DensePlan pl;
  if (int rc = plan_dense(v, dev, nullptr, nullptr, m, n, k, static_cast<size_t>(-1), &pl); rc != 0) return rc;
  std::memset(out, 0, sizeof(*out));
  out->path = !pl.tensor_core ? B200_LAUNCHED_SIMT : (pl.kernel.pair ? B200_LAUNCHED_TCGEN05_PAIR : B200_LAUNCHED_TCGEN05);
  out->grid = pl.grid;
  out->tile_rows = pl.tensor_core ? pl.tile_rows : 4;
  out->tile_cols = pl.tensor_core ? pl.tile_cols : 64;
  out->group_m = pl.tensor_core ? pl.group_m : 0;
  out->split_k = pl.slices;
  out->tail_units = pl.tail_units;
  if (pl.mix_total_wide >= 0) out->tiles_384 = pl.mix_rows_hi * pl.mix_tq_hi + (pl.tiles_m - pl.mix_rows_hi) * pl.mix_tq_lo;
  return 0;
}

extern "C" int b200_int4_gemms_launch_dense(const b200_gemm_variant* v, int device_index,
                                            uintptr_t stream_handle, const void* a, const void* b,
                                            const void* a_scale, const void* b_scale, void* c,
                                            void* workspace, size_t workspace_bytes, int32_t m,
                                            int32_t n, int32_t k) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  if (int rc = check_variant(v); rc != 0) return rc;
  if (a == nullptr || b == nullptr || c == nullptr) return fail("a, b and c pointers must be non-null");
  if (v->out_dtype != B200_OUT_S32 && (a_scale == nullptr || b_scale == nullptr))
    return fail("a_scale and b_scale pointers must be non-null");
  if (m <= 0 || n <= 0 || k <= 0) return fail("m, n and k must be positive");
  const bool int4 = v->dtype == B200_DTYPE_INT4;
  if (int4 && k >= 131072) return fail("int4 path supports k < 131072 (accumulator headroom of the 16x operand encoding)");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_handle);

  const bool swiglu = v->epilogue == B200_EPILOGUE_SWIGLU;
  const int b_cols = swiglu ? 2 * n : n;
  const int kb = int4 ? (k + 1) / 2 : k;
  const bool a_t = (v->layout == B200_LAYOUT_TN || v->layout == B200_LAYOUT_TT);
  const bool b_t = (v->layout == B200_LAYOUT_NT || v->layout == B200_LAYOUT_TT);
  const int sc_mode = (v->scale_mode == B200_SCALE_SUBCHANNEL) ? SCALE_SC : SCALE_PC;
  const int scale_cols = sc_mode == SCALE_SC ? (k + v->subchannel - 1) / v->subchannel : 1;

  DensePlan pl;
  const size_t usable_workspace = (workspace != nullptr && aligned16(workspace)) ? workspace_bytes : 0;
  if (int rc = plan_dense(v, dev, a, b, m, n, k, usable_workspace, &pl); rc != 0) return rc;

  if (!pl.tensor_core) {
    SimtParams sp{};
    sp.mode = MODE_DENSE;
    sp.int4 = int4;
    sp.a_transposed = a_t;
    sp.b_transposed = b_t;
    sp.scale_mode = sc_mode;
    sp.subchannel = v->subchannel;
    sp.scale_cols = scale_cols;
    sp.epilogue = v->epilogue;
    sp.out_dtype = v->out_dtype;
    sp.M = m;
    sp.N = n;
    sp.K = k;
    sp.b_cols = b_cols;
    sp.kb = kb;
    sp.a = static_cast<const uint8_t*>(a);
    sp.b = static_cast<const uint8_t*>(b);
    sp.a_scale = static_cast<const __nv_bfloat16*>(a_scale);
    sp.b_scale = static_cast<const __nv_bfloat16*>(b_scale);
    sp.out = c;
    g_last_path = B200_LAUNCHED_SIMT;
    return launch_simt(sp, m, 1, stream);
  }

  const bool split = pl.slices > 1;
  if (split) {
    const size_t need = static_cast<size_t>(pl.slices) * m * n * 4u;
    if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace))
      return fail("split_k > 1 needs a 16-byte aligned workspace of b200_int4_gemms_dense_workspace_bytes(...) bytes");
  }

  CUtensorMap ta, tb;
  if (int4) {
    if (a_t) {
      if (int rc = make_map_2d(&ta, a, m, kb, m, NBLK, BK / 2, 0, "A"); rc != 0) return rc;
    } else {
      // A through TMEM: a thread of the unpack warps reads one 64-byte row of the staging tile, so TMA writes the tile
      // with the 64-byte swizzle
      const int a_swizzle = pl.kernel.flavor == FLAVOR_TMEM_A ? 64 : 0;
      if (int rc = make_map_2d(&ta, a, kb, m, kb, BK / 2, BM, a_swizzle, "A"); rc != 0) return rc;
    }
    if (b_t) {
      if (int rc = make_map_2d(&tb, b, kb, b_cols, kb, BK / 2, NBLK, 0, "B"); rc != 0) return rc;
    } else {
      if (int rc = make_map_2d(&tb, b, b_cols, kb, b_cols, NBLK, BK / 2, 0, "B"); rc != 0) return rc;
    }
  } else {
    if (a_t) {
      if (int rc = make_map_2d(&ta, a, m, kb, m, NBLK, BK, 128, "A"); rc != 0) return rc;
    } else {
      if (int rc = make_map_2d(&ta, a, kb, m, kb, BK, BM, 128, "A"); rc != 0) return rc;
    }
    if (b_t) {
      if (int rc = make_map_2d(&tb, b, kb, b_cols, kb, BK, NBLK, 128, "B"); rc != 0) return rc;
    } else {
      if (int rc = make_map_2d(&tb, b, b_cols, kb, b_cols, NBLK, BK, 128, "B"); rc != 0) return rc;
    }
  }

  GemmParams p{};
  p.mode = MODE_DENSE;
  p.M = m;
  p.N = n;
  p.K = k;
  p.tile_cols = pl.tile_cols;
  p.tiles_n = pl.tiles_n;
  p.tiles_m = pl.tiles_m;
  p.k_slices = pl.slices;
  p.k_per_slice = pl.k_per_slice;
  p.num_tiles = p.tiles_m * p.tiles_n * pl.slices;
  p.mix_total_wide = pl.mix_total_wide;
  if (pl.mix_total_wide >= 0) {
    p.mix_rows_hi = pl.mix_rows_hi;
    p.mix_wide_hi = pl.mix_wide_hi;
    p.mix_wide_lo = pl.mix_wide_lo;
    p.mix_tq_hi = pl.mix_tq_hi;
    p.mix_tq_lo = pl.mix_tq_lo;
    p.num_tiles = pl.mix_total_wide + pl.mix_rows_hi * pl.mix_tq_hi + (p.tiles_m - pl.mix_rows_hi) * pl.mix_tq_lo;
  }
  p.group_m = pl.group_m;
  p.gate_col_offset = swiglu ? n : NBLK;
  p.ldc = n;
  p.subchannel = sc_mode == SCALE_SC ? v->subchannel : 0;
  p.scale_cols = scale_cols;
  p.lds_b = b_cols;
  p.a_scale = static_cast<const __nv_bfloat16*>(a_scale);
  p.b_scale = static_cast<const __nv_bfloat16*>(b_scale);
  p.out = split ? workspace : c;
  p.status = dev->status_dev;
  if (pl.tail_units > 0) {
    p.tail_units = pl.tail_units;
    p.tail_split = pl.tail_split;
    p.tail_waves = pl.tail_waves;
    p.tail_rest = pl.tail_rest;
    p.tail_kb_per_tile = (k + BK - 1) / BK;
    p.tail_flags = static_cast<int*>(workspace);
    p.tail_partials = reinterpret_cast<int*>(static_cast<char*>(workspace) + kTailFlagBytes);
    if (!workspace_seen_before(workspace, workspace_bytes, device_index)) {
      cudaError_t err = cudaMemsetAsync(p.tail_flags, 0, kTailFlagBytes, stream);
      if (err != cudaSuccess) return fail_cuda("cudaMemsetAsync(balanced-tail flags)", err);
    }
  }
  CUtensorMap tc;
  std::memset(&tc, 0, sizeof(tc));
  if (!split) {
    if (int rc = make_output_map(&tc, c, v->out_dtype, m, n, &p.tma_store); rc != 0) return rc;
  }
  int rc = launch_tc(pl.kernel, ta, tb, tc, p, pl.grid, stream);
  if (rc < 0) return fail("internal: no tcgen05 instantiation for this variant");
  if (rc != 0) return rc;
  g_last_path = pl.kernel.pair ? B200_LAUNCHED_TCGEN05_PAIR : B200_LAUNCHED_TCGEN05;
  if (split) {
    const long long items = (n % 4 == 0) ? static_cast<long long>(m) * n / 4 : static_cast<long long>(m) * n;
    long long blocks = (items + 255) / 256;
    const long long cap = static_cast<long long>(dev->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    splitk_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        workspace, static_cast<float*>(c), p.a_scale, p.b_scale, m, n, pl.slices, pl.integer_partials ? 1 : 0);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail_cuda("split-K reduction kernel launch", err);
  }
  return 0;
}

namespace {

// Grouped forward launch.  num_tasks_dev == nullptr: the host knows the task count (num_tasks).  Otherwise
// the task arrays hold num_tasks entries of capacity and the device-side count says how many are real.
int launch_ragged_fwd_impl(
    const b200_gemm_variant* v, int device_index, uintptr_t stream_handle, const void* lhs,
    const void* rhs, const void* lhs_scale, const void* rhs_scale, const int64_t* task_group_ids,
    const int64_t* task_block_starts, const int64_t* task_actual_starts,
    const int64_t* task_actual_ends, const int32_t* num_tasks_dev, const int32_t* overflow_dev, void* out,
    int32_t m, int32_t n, int32_t k_packed, int32_t scale_cols, int32_t num_tasks, int32_t groups,
    int32_t block_rows) {
  if (int rc = check_variant(v); rc != 0) return rc;
  if (v->dtype != B200_DTYPE_INT4) return fail("ragged kernels take packed int4 operands");
  if (v->epilogue != B200_EPILOGUE_NONE) return fail("ragged kernels have no fused activation");
  if (v->out_dtype == B200_OUT_S32) return fail("ragged kernels store bf16 or float32");
  if (lhs == nullptr || rhs == nullptr || lhs_scale == nullptr || rhs_scale == nullptr ||
      task_group_ids == nullptr || task_block_starts == nullptr || task_actual_starts == nullptr ||
      task_actual_ends == nullptr || out == nullptr)
    return fail("ragged forward kernel pointers must be non-null");
  if (m <= 0 || n <= 0 || k_packed <= 0 || groups <= 0) return fail("m, n, k_packed and groups must be positive");
  if (num_tasks < 0) return fail("num_tasks must be non-negative");
  if (block_rows <= 0 || block_rows > 2 * BM) return fail("block_rows must be in [1, 256]");
  if (k_packed >= 65536) return fail("int4 path supports k < 131072");
  if (num_tasks == 0) return 0;
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_handle);

  const bool a_t = (v->layout == B200_LAYOUT_TN || v->layout == B200_LAYOUT_TT);
  const bool b_t = (v->layout == B200_LAYOUT_NT || v->layout == B200_LAYOUT_TT);
  const int sc_mode = (v->scale_mode == B200_SCALE_SUBCHANNEL) ? SCALE_SC : SCALE_PC;
  const int k = 2 * k_packed;
  if (sc_mode == SCALE_SC && scale_cols != (k + v->subchannel - 1) / v->subchannel)
    return fail("scale_cols does not match ceil(K / subchannel)");

  // Tasks of more than 128 rows run on CTA pairs: rank 0 takes the first 128 rows of the block, rank 1 the rest.
  // A transposed lhs [Kb, M] puts the task's first row (a multiple of the align_tile the tasks were built with) on
  // the TMA x axis, which wants multiples of 16 bytes: it is taken when the caller states that alignment in the
  // variant (the kernel skips and reports a task that breaks it); rhs may be [G, Kb, N] or [G, N, Kb]
  TcLaunch tl{true, a_t, !b_t, false, sc_mode, EPI_NONE, v->out_dtype};
  tl.pair = block_rows > BM;
  const bool pair_ok = !tl.pair || sc_mode == SCALE_PC || v->subchannel >= BK;
  const bool lhs_ok = a_t ? (v->task_align > 0 && v->task_align % 16 == 0 && block_rows % 16 == 0 && m % 16 == 0 && !tl.pair)
                          : (k_packed % 16 == 0);
  bool tc_ok = lhs_ok && pair_ok && tc_has(tl) && aligned16(lhs) && aligned16(rhs) && (b_t ? k_packed % 16 == 0 : n % 16 == 0);
  if (v->path == B200_PATH_SIMT) tc_ok = false;
  if (v->path == B200_PATH_TCGEN05 && !tc_ok)
    return fail("the tcgen05 ragged forward kernel needs 16-byte aligned operands and operand pitches that are multiples of 16 "
                "bytes, for a transposed lhs (TN / TT) task starts stated as multiples of 16 rows (variant.task_align) and "
                "tasks of at most 128 rows, and for block_rows > 128 per-channel scales or K-groups of at least 128");

  if (!tc_ok) {
    SimtParams sp{};
    sp.mode = MODE_RAGGED_FWD;
    sp.int4 = 1;
    sp.a_transposed = a_t;
    sp.b_transposed = b_t;
    sp.scale_mode = sc_mode;
    sp.subchannel = v->subchannel;
    sp.scale_cols = sc_mode == SCALE_SC ? scale_cols : 1;
    sp.epilogue = EPI_NONE;
    sp.out_dtype = v->out_dtype;
    sp.M = m;
    sp.N = n;
    sp.K = k;
    sp.b_cols = n;
    sp.kb = k_packed;
    sp.num_groups = groups;
    sp.num_tasks = num_tasks;
    sp.a = static_cast<const uint8_t*>(lhs);
    sp.b = static_cast<const uint8_t*>(rhs);
    sp.a_scale = static_cast<const __nv_bfloat16*>(lhs_scale);
    sp.b_scale = static_cast<const __nv_bfloat16*>(rhs_scale);
    sp.task_group_ids = reinterpret_cast<const long long*>(task_group_ids);
    sp.task_actual_starts = reinterpret_cast<const long long*>(task_actual_starts);
    sp.task_actual_ends = reinterpret_cast<const long long*>(task_actual_ends);
    sp.out = out;
    // with a device-side count the padding entries are empty tasks (actual_start == actual_end): no rows
    g_last_path = B200_LAUNCHED_SIMT;
    return launch_simt(sp, block_rows, num_tasks, stream);
  }

  if (tl.pair && (v->a_operand == B200_A_OPERAND_TMEM || (v->a_operand == B200_A_OPERAND_AUTO && k >= 48 * BK))) {
    TcLaunch through_tmem = tl;
    through_tmem.flavor = FLAVOR_TMEM_A;
    if (tc_has(through_tmem)) tl = through_tmem;
  }
  CUtensorMap ta, tb;
  if (a_t) {
    if (int rc = make_map_2d(&ta, lhs, m, k_packed, m, NBLK, BK / 2, 0, "lhs"); rc != 0) return rc;
  } else {
    if (int rc = make_map_2d(&ta, lhs, k_packed, m, k_packed, BK / 2, BM, tl.flavor == FLAVOR_TMEM_A ? 64 : 0, "lhs"); rc != 0) return rc;
  }
  if (b_t) {
    if (int rc = make_map_2d(&tb, rhs, k_packed, static_cast<uint64_t>(groups) * n, k_packed, BK / 2, NBLK, 0, "rhs"); rc != 0)
      return rc;
  } else {
    if (int rc = make_map_2d(&tb, rhs, n, static_cast<uint64_t>(groups) * k_packed, n, NBLK, BK / 2, 0, "rhs"); rc != 0)
      return rc;
  }
  // wide tiles (256 rows x 512 columns per pair), by the rule of the dense launches: a wide tile takes 0.9 of the
  // time of the two it replaces (with a device-side task count, num_tasks is the capacity of the arrays)
  int tile_cols = BN;
  if (tl.pair && (tl.flavor == FLAVOR_PLAIN || tl.flavor == FLAVOR_TMEM_A) && v->wide_tiles != B200_WIDE_OFF && dev->max_pair_clusters > 0) {
    TcLaunch wide = tl;
    wide.flavor = FLAVOR_WIDE;
    const long long units = dev->max_pair_clusters;
    const long long narrow_waves = (static_cast<long long>(num_tasks) * ((n + BN - 1) / BN) + units - 1) / units;
    const long long wide_waves = (static_cast<long long>(num_tasks) * ((n + 2 * BN - 1) / (2 * BN)) + units - 1) / units;
    if (tc_has(wide) && (v->wide_tiles == B200_WIDE_ON || 18 * wide_waves < 10 * narrow_waves)) {
      tl = wide;
      tile_cols = 2 * BN;
      // the lhs map of the A-through-TMEM kernel is swizzled; the wide kernel stages A like the plain one
      if (int rc = make_map_2d(&ta, lhs, k_packed, m, k_packed, BK / 2, BM, 0, "lhs"); rc != 0) return rc;
    }
  }
  GemmParams p{};
  p.mode = MODE_RAGGED_FWD;
  p.M = m;
  p.N = n;
  p.K = k;
  p.tile_cols = tile_cols;
  p.tiles_m = num_tasks;
  p.tiles_n = (n + tile_cols - 1) / tile_cols;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.group_m = 1;
  p.gate_col_offset = NBLK;
  p.ldc = n;
  p.subchannel = sc_mode == SCALE_SC ? v->subchannel : 0;
  p.scale_cols = sc_mode == SCALE_SC ? scale_cols : 1;
  p.lds_b = n;
  p.num_groups = groups;
  p.rows_per_group_b = b_t ? n : k_packed;  // rows of the stacked rhs map per group
  p.task_group_ids = reinterpret_cast<const long long*>(task_group_ids);
  p.task_block_starts = reinterpret_cast<const long long*>(task_block_starts);
  p.task_actual_starts = reinterpret_cast<const long long*>(task_actual_starts);
  p.task_actual_ends = reinterpret_cast<const long long*>(task_actual_ends);
  p.num_tasks_dev = num_tasks_dev;
  p.overflow_dev = overflow_dev;
  p.a_scale = static_cast<const __nv_bfloat16*>(lhs_scale);
  p.b_scale = static_cast<const __nv_bfloat16*>(rhs_scale);
  p.out = out;
  p.status = dev->status_dev;
  CUtensorMap tc;
  if (int rc = make_output_map(&tc, out, v->out_dtype, m, n, &p.tma_store); rc != 0) return rc;
  const int cta_per_tile = tl.pair ? 2 : 1;
  const int max_units = tl.pair ? dev->max_pair_clusters : dev->sm_count;
  const int grid = (p.num_tiles < max_units ? p.num_tiles : max_units) * cta_per_tile;
  int rc = launch_tc(tl, ta, tb, tc, p, grid, stream);
  if (rc < 0) return fail("internal: no tcgen05 instantiation for this variant");
  if (rc == 0) g_last_path = tl.pair ? B200_LAUNCHED_TCGEN05_PAIR : B200_LAUNCHED_TCGEN05;
  return rc;
}

}  // namespace

extern "C" int b200_int4_gemms_launch_ragged_fwd(
    const b200_gemm_variant* v, int device_index, uintptr_t stream_handle, const void* lhs,
    const void* rhs, const void* lhs_scale, const void* rhs_scale, const int64_t* task_group_ids,
    const int64_t* task_block_starts, const int64_t* task_actual_starts,
    const int64_t* task_actual_ends, void* out, int32_t m, int32_t n, int32_t k_packed,
    int32_t scale_cols, int32_t num_tasks, int32_t groups, int32_t block_rows) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  return launch_ragged_fwd_impl(v, device_index, stream_handle, lhs, rhs, lhs_scale, rhs_scale, task_group_ids,
                                task_block_starts, task_actual_starts, task_actual_ends, nullptr, nullptr, out, m,
                                n, k_packed, scale_cols, num_tasks, groups, block_rows);
}

extern "C" int b200_int4_gemms_launch_ragged_fwd_device_tasks(
    const b200_gemm_variant* v, int device_index, uintptr_t stream_handle, const void* lhs,
    const void* rhs, const void* lhs_scale, const void* rhs_scale, const int64_t* task_group_ids,
    const int64_t* task_block_starts, const int64_t* task_actual_starts,
    const int64_t* task_actual_ends, const int32_t* num_tasks_dev, const int32_t* overflow_dev, void* out,
    int32_t m, int32_t n, int32_t k_packed, int32_t scale_cols, int32_t max_tasks, int32_t groups,
    int32_t block_rows) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  if (num_tasks_dev == nullptr) return fail("num_tasks_dev must be non-null");
  return launch_ragged_fwd_impl(v, device_index, stream_handle, lhs, rhs, lhs_scale, rhs_scale, task_group_ids,
                                task_block_starts, task_actual_starts, task_actual_ends, num_tasks_dev, overflow_dev,
                                out, m, n, k_packed, scale_cols, max_tasks, groups, block_rows);
}

extern "C" int b200_int4_gemms_group_info(int device_index, uintptr_t stream_handle, const int64_t* group_sizes,
                                          int32_t groups, int32_t tile, int32_t align, int64_t* task_group_ids,
                                          int64_t* task_block_starts, int64_t* task_actual_starts,
                                          int64_t* task_actual_ends, int32_t max_tasks, int32_t* num_tasks_dev,
                                          int32_t* overflow_dev) {
  g_last_error.clear();
  if (group_sizes == nullptr || task_group_ids == nullptr || task_block_starts == nullptr ||
      task_actual_starts == nullptr || task_actual_ends == nullptr || num_tasks_dev == nullptr || overflow_dev == nullptr)
    return fail("group-info pointers must be non-null");
  if (groups <= 0 || max_tasks <= 0) return fail("groups and max_tasks must be positive");
  if (tile <= 0 || align <= 0 || tile % align != 0) return fail("tile must be a positive multiple of align");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  group_info_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream_handle)>>>(
      reinterpret_cast<const long long*>(group_sizes), groups, tile, align, reinterpret_cast<long long*>(task_group_ids),
      reinterpret_cast<long long*>(task_block_starts), reinterpret_cast<long long*>(task_actual_starts),
      reinterpret_cast<long long*>(task_actual_ends), max_tasks, num_tasks_dev, overflow_dev);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("group-info kernel launch", err);
  return 0;
}

extern "C" int b200_int4_gemms_quantize(int device_index, uintptr_t stream_handle, const void* src_bf16, void* dst,
                                        int64_t rows, int64_t cols, int32_t bits, float scale) {
  g_last_error.clear();
  if (src_bf16 == nullptr || dst == nullptr) return fail("src and dst pointers must be non-null");
  if (rows < 0 || cols < 0) return fail("rows and cols must be non-negative");
  if (bits != 4 && bits != 8) return fail("bits must be 4 or 8");
  if (!(scale > 0.f)) return fail("scale must be positive");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  const long long total = rows * ((cols + 7) / 8);
  if (total == 0) return 0;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  quantize_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_handle)>>>(
      static_cast<const __nv_bfloat16*>(src_bf16), static_cast<uint8_t*>(dst), rows, cols, bits, scale);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("quantize kernel launch", err);
  return 0;
}

extern "C" int b200_int4_gemms_repack_tokens(int device_index, uintptr_t stream_handle, const void* src, void* dst,
                                             int64_t rows, int64_t cols) {
  g_last_error.clear();
  if (src == nullptr || dst == nullptr) return fail("src and dst pointers must be non-null");
  if (rows < 0 || cols < 0 || cols % 2 != 0) return fail("rows must be non-negative and cols a non-negative even number");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  const long long total = ((rows + 1) / 2) * ((cols + 7) / 8);
  if (total == 0) return 0;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  repack_tokens_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_handle)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("token repack kernel launch", err);
  return 0;
}

namespace {

// Grouped backward launch.  group_starts == nullptr: operands stacked per group ([G, k_packed, M] /
// [G, k_packed, N], or [G, M, k_packed] for a K-major lhs).  Otherwise: flat token-packed operands
// ([k_packed, M] / [k_packed, N] over all tokens) and group_starts[g] = first token of group g.
int launch_ragged_bwd_impl(const b200_gemm_variant* v, int device_index, uintptr_t stream_handle,
                           const void* lhs, const void* rhs, const void* lhs_scale, const void* rhs_scale,
                           const int64_t* group_sizes, const long long* group_starts, void* out, int32_t m,
                           int32_t n, int32_t k_packed, int32_t scale_cols, int32_t groups,
                           DeviceState* prepared = nullptr) {
  const bool flat = group_starts != nullptr;
  if (int rc = check_variant(v); rc != 0) return rc;
  if (v->dtype != B200_DTYPE_INT4) return fail("ragged kernels take packed int4 operands");
  if (v->epilogue != B200_EPILOGUE_NONE) return fail("ragged kernels have no fused activation");
  if (v->out_dtype != B200_OUT_F32) return fail("ragged backward stores float32");
  if (lhs == nullptr || rhs == nullptr || lhs_scale == nullptr || rhs_scale == nullptr ||
      group_sizes == nullptr || out == nullptr)
    return fail("ragged backward kernel pointers must be non-null");
  if (m <= 0 || n <= 0 || k_packed <= 0 || groups <= 0) return fail("m, n, k_packed and groups must be positive");
  // stacked operands: k_packed bounds one group's reduction; flat operands: it is the whole token axis,
  // and a single group longer than the accumulator headroom is the caller's to avoid
  if (!flat && k_packed >= 65536) return fail("int4 path supports k < 131072");
  DeviceState* dev = prepared;  // a caller that has done its own device set-up passes it in
  if (dev == nullptr) {
    if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_handle);

  const bool a_t = (v->layout == B200_LAYOUT_TN || v->layout == B200_LAYOUT_TT);
  const bool b_t = (v->layout == B200_LAYOUT_NT || v->layout == B200_LAYOUT_TT);
  const int sc_mode = (v->scale_mode == B200_SCALE_SUBCHANNEL) ? SCALE_SC : SCALE_PC;
  const int k = 2 * k_packed;
  if (flat && (!a_t || b_t)) return fail("flat backward operands are token-major: layout TN");
  if (flat && sc_mode != SCALE_PC) return fail("flat backward operands support per-channel scales");
  if (sc_mode == SCALE_SC && scale_cols != (k + v->subchannel - 1) / v->subchannel)
    return fail("scale_cols does not match ceil(K / subchannel)");

  TcLaunch tl{true, a_t, !b_t, true, sc_mode, EPI_NONE, OUT_F32};
  bool tc_ok = tc_has(tl) && aligned16(lhs) && aligned16(rhs) && ((a_t ? m : k_packed) % 16 == 0) &&
               ((b_t ? k_packed : n) % 16 == 0);
  // CTA pairs (256-row tiles) where a paired kernel exists and the rows fill them: a third less operand
  // traffic through each SM's shared memory, which this kernel shares with its fp32 output staging
  if (tc_ok && dev->max_pair_clusters > 0 && m % (2 * BM) == 0 && v->cta_group != B200_CTA_GROUP_SINGLE) {
    TcLaunch pl = tl;
    pl.pair = true;
    const bool sc_ok = sc_mode == SCALE_PC || v->subchannel >= BK;  // paired kernels hand accumulators over per K block
    if (sc_ok && tc_has(pl)) tl = pl;
  }
  if (v->path == B200_PATH_SIMT) tc_ok = false;
  if (v->path == B200_PATH_TCGEN05 && !tc_ok)
    return fail("the tcgen05 ragged backward kernel needs 16-byte aligned operands, operand pitches that are multiples of 16 bytes and, for a K-major rhs (NT / TT), per-channel scales");

  if (!tc_ok) {
    SimtParams sp{};
    sp.mode = MODE_RAGGED_BWD;
    sp.int4 = 1;
    sp.a_transposed = a_t;
    sp.b_transposed = b_t;
    sp.scale_mode = sc_mode;
    sp.subchannel = v->subchannel;
    sp.scale_cols = sc_mode == SCALE_SC ? scale_cols : 1;
    sp.epilogue = EPI_NONE;
    sp.out_dtype = OUT_F32;
    sp.M = m;
    sp.N = n;
    sp.K = k;
    sp.b_cols = n;
    sp.kb = k_packed;
    sp.num_groups = groups;
    sp.a = static_cast<const uint8_t*>(lhs);
    sp.b = static_cast<const uint8_t*>(rhs);
    sp.a_scale = static_cast<const __nv_bfloat16*>(lhs_scale);
    sp.b_scale = static_cast<const __nv_bfloat16*>(rhs_scale);
    sp.group_sizes = reinterpret_cast<const long long*>(group_sizes);
    sp.group_starts = group_starts;
    sp.out = out;
    g_last_path = B200_LAUNCHED_SIMT;
    return launch_simt(sp, m, groups, stream);
  }

  const uint64_t k_rows = flat ? static_cast<uint64_t>(k_packed) : static_cast<uint64_t>(groups) * k_packed;
  CUtensorMap ta, tb;
  if (a_t) {
    if (int rc = make_map_2d(&ta, lhs, m, k_rows, m, NBLK, BK / 2, 0, "lhs"); rc != 0)
      return rc;
  } else {
    if (int rc = make_map_2d(&ta, lhs, k_packed, static_cast<uint64_t>(groups) * m, k_packed, BK / 2, BM, 0, "lhs"); rc != 0)
      return rc;
  }
  if (b_t) {
    if (int rc = make_map_2d(&tb, rhs, k_packed, static_cast<uint64_t>(groups) * n, k_packed, BK / 2, NBLK, 0, "rhs"); rc != 0)
      return rc;
  } else {
    if (int rc = make_map_2d(&tb, rhs, n, k_rows, n, NBLK, BK / 2, 0, "rhs"); rc != 0)
      return rc;
  }
  GemmParams p{};
  p.mode = MODE_RAGGED_BWD;
  p.group_starts = group_starts;
  p.M = m;
  p.N = n;
  p.K = k;
  p.tile_cols = BN;
  p.tiles_m = (m + (tl.pair ? 2 * BM : BM) - 1) / (tl.pair ? 2 * BM : BM);
  p.tiles_n = (n + BN - 1) / BN;
  p.num_tiles = groups * p.tiles_m * p.tiles_n;
  p.group_m = 1;
  p.gate_col_offset = NBLK;
  p.ldc = n;
  p.subchannel = sc_mode == SCALE_SC ? v->subchannel : 0;
  p.scale_cols = sc_mode == SCALE_SC ? scale_cols : 1;
  p.lds_b = n;
  p.num_groups = groups;
  p.rows_per_group_a = a_t ? k_packed : m;
  p.rows_per_group_b = b_t ? n : k_packed;
  p.group_sizes = reinterpret_cast<const long long*>(group_sizes);
  p.a_scale = static_cast<const __nv_bfloat16*>(lhs_scale);
  p.b_scale = static_cast<const __nv_bfloat16*>(rhs_scale);
  p.out = out;
  p.status = dev->status_dev;
  CUtensorMap tc;
  if (int rc = make_output_map(&tc, out, OUT_F32, static_cast<uint64_t>(groups) * m, n, &p.tma_store); rc != 0) return rc;
  const int units = tl.pair ? dev->max_pair_clusters : dev->sm_count;
  const int grid = (p.num_tiles < units ? p.num_tiles : units) * (tl.pair ? 2 : 1);
  int rc = launch_tc(tl, ta, tb, tc, p, grid, stream);
  if (rc < 0) return fail("internal: no tcgen05 instantiation for this variant");
  if (rc == 0) g_last_path = tl.pair ? B200_LAUNCHED_TCGEN05_PAIR : B200_LAUNCHED_TCGEN05;
  return rc;
}

int launch_group_starts(const int64_t* group_sizes, long long* starts, int groups, cudaStream_t stream) {
  group_starts_kernel<<<1, 1024, 0, stream>>>(reinterpret_cast<const long long*>(group_sizes), starts, groups);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("group-start scan launch", err);
  return 0;
}

}  // namespace

extern "C" int b200_int4_gemms_launch_ragged_bwd(const b200_gemm_variant* v, int device_index,
                                                 uintptr_t stream_handle, const void* lhs,
                                                 const void* rhs, const void* lhs_scale,
                                                 const void* rhs_scale, const int64_t* group_sizes,
                                                 void* out, int32_t m, int32_t n, int32_t k_packed,
                                                 int32_t scale_cols, int32_t groups) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  return launch_ragged_bwd_impl(v, device_index, stream_handle, lhs, rhs, lhs_scale, rhs_scale, group_sizes,
                                nullptr, out, m, n, k_packed, scale_cols, groups);
}

extern "C" size_t b200_int4_gemms_ragged_bwd_flat_workspace_bytes(int32_t groups) {
  return groups > 0 ? (static_cast<size_t>(groups) + 1) * sizeof(long long) : 0;
}

extern "C" int b200_int4_gemms_launch_ragged_bwd_flat(const b200_gemm_variant* v, int device_index,
                                                      uintptr_t stream_handle, const void* lhs,
                                                      const void* rhs, const void* lhs_scale,
                                                      const void* rhs_scale, const int64_t* group_sizes,
                                                      void* out, void* workspace, size_t workspace_bytes,
                                                      int32_t m, int32_t n, int64_t tokens, int32_t groups) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  if (tokens <= 0 || groups <= 0) return fail("tokens and groups must be positive");
  if ((tokens + 1) / 2 > 0x7FFFFFFF) return fail("too many tokens for one launch");
  if (group_sizes == nullptr) return fail("ragged backward kernel pointers must be non-null");
  if (workspace == nullptr || workspace_bytes < b200_int4_gemms_ragged_bwd_flat_workspace_bytes(groups) ||
      (reinterpret_cast<uintptr_t>(workspace) & 7u) != 0)
    return fail("workspace must be 8-byte aligned and hold b200_int4_gemms_ragged_bwd_flat_workspace_bytes(groups) bytes");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  long long* starts = static_cast<long long*>(workspace);
  if (int rc = launch_group_starts(group_sizes, starts, groups, reinterpret_cast<cudaStream_t>(stream_handle)); rc != 0) return rc;
  return launch_ragged_bwd_impl(v, device_index, stream_handle, lhs, rhs, lhs_scale, rhs_scale, group_sizes, starts,
                                out, m, n, static_cast<int32_t>((tokens + 1) / 2), 1, groups);
}

// ---------------------------------------------------------------------------------------------
// Flat grouped backward without a caller-provided workspace and without any allocation.
// ---------------------------------------------------------------------------------------------
namespace {

// The group-start scan's scratch, for callers that cannot bring device memory of their own.  One
// array per loaded library image and device, shared by every call of the entry point below: calls
// that may run at the same time (different streams, different host threads) would overwrite each
// other's group starts.  Every call rewrites entries [0, groups] before its GEMM kernel reads them,
// so nothing in it has to be zero and stale contents of an earlier call do no harm.
static __device__ __align__(256) long long g_static_group_starts[B200_STATIC_SCRATCH_MAX_GROUPS + 1];

struct StaticScratchState {
  bool ready = false;
  DeviceState view;             // SM count for the grid; status word borrowed when the device has one
  long long* starts = nullptr;  // device address of g_static_group_starts on this device
};
StaticScratchState g_static_devices[kMaxDevices];
std::mutex g_static_mutex;

// First call per device: look the array's address up and give the one tensor-core kernel this entry
// point launches its shared-memory size.  No allocation: unlike ensure_device, no status word is made.
int ensure_static_scratch(int device_index, StaticScratchState** out) {
  if (device_index < 0 || device_index >= kMaxDevices) return fail("device_index out of range");
  cudaError_t err = cudaSetDevice(device_index);
  if (err != cudaSuccess) return fail_cuda("cudaSetDevice", err);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticScratchState& st = g_static_devices[device_index];
  if (!st.ready) {
    int major = 0, sms = 0;
    err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_index);
    if (err != cudaSuccess) return fail_cuda("cudaDeviceGetAttribute(compute capability)", err);
    if (major != 10) return fail("this library holds sm_100a kernels only");
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_index);
    if (err != cudaSuccess) return fail_cuda("cudaDeviceGetAttribute(SM count)", err);
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_group_starts);
    if (err != cudaSuccess) return fail_cuda("cudaGetSymbolAddress(static group-start scratch)", err);
    if (address == nullptr) return fail("static group-start scratch has no device address");
    // the one tensor-core kernel this entry point launches: same set-up and register check as ensure_device
    const TcKernelInfo* kernel = tc_find(TcLaunch{true, true, true, true, SCALE_PC, EPI_NONE, OUT_F32, false});
    if (kernel == nullptr) return fail("internal: the flat backward kernel is not part of this build");
    if (int rc = prepare_kernel(*kernel); rc != 0) return rc;
    st.view.sm_count = sms;
    st.view.cc_major = major;
    st.view.max_pair_clusters = 0;  // this entry point never launches a CTA-pair kernel
    st.starts = static_cast<long long*>(address);
    st.ready = true;
  }
  // time-outs of bounded device waits are recorded only if another entry point has given the device a status word
  {
    std::lock_guard<std::mutex> dev_lock(g_device_mutex);
    st.view.status_dev = g_devices[device_index].ready ? g_devices[device_index].status_dev : nullptr;
  }
  *out = &st;
  return 0;
}

}  // namespace

extern "C" int b200_int4_gemms_launch_ragged_bwd_flat_static(const b200_gemm_variant* v, int device_index,
                                                             uintptr_t stream_handle, const void* lhs,
                                                             const void* rhs, const void* lhs_scale,
                                                             const void* rhs_scale, const int64_t* group_sizes,
                                                             void* out, int32_t m, int32_t n, int64_t tokens,
                                                             int32_t groups) {
  g_last_error.clear();
  g_last_path = B200_LAUNCHED_NOTHING;
  if (tokens <= 0 || groups <= 0) return fail("tokens and groups must be positive");
  if (groups > B200_STATIC_SCRATCH_MAX_GROUPS)
    return fail("the built-in scratch holds the starts of at most " + std::to_string(B200_STATIC_SCRATCH_MAX_GROUPS) +
                " groups; got " + std::to_string(groups) +
                " (use b200_int4_gemms_launch_ragged_bwd_flat with a workspace of your own)");
  if ((tokens + 1) / 2 > 0x7FFFFFFF) return fail("too many tokens for one launch");
  if (group_sizes == nullptr) return fail("ragged backward kernel pointers must be non-null");
  StaticScratchState* st = nullptr;
  if (int rc = ensure_static_scratch(device_index, &st); rc != 0) return rc;
  if (int rc = launch_group_starts(group_sizes, st->starts, groups, reinterpret_cast<cudaStream_t>(stream_handle)); rc != 0) return rc;
  return launch_ragged_bwd_impl(v, device_index, stream_handle, lhs, rhs, lhs_scale, rhs_scale, group_sizes, st->starts,
                                out, m, n, static_cast<int32_t>((tokens + 1) / 2), 1, groups, &st->view);
}

extern "C" int b200_int4_gemms_unpack_int4(int device_index, uintptr_t stream_handle,
                                           const void* packed, void* out_int8, int64_t rows,
                                           int64_t cols_packed) {
  g_last_error.clear();
  if (packed == nullptr || out_int8 == nullptr) return fail("packed and out_int8 pointers must be non-null");
  if (rows < 0 || cols_packed < 0) return fail("rows and cols_packed must be non-negative");
  if (!aligned16(packed) || !aligned16(out_int8)) return fail("packed and out_int8 must be 16-byte aligned");
  DeviceState* dev = nullptr;
  if (int rc = ensure_device(device_index, &dev); rc != 0) return rc;
  const long long total = rows * cols_packed;
  if (total == 0) return 0;
  long long blocks = (total / 16 + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  unpack_int4_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream_handle)>>>(
      static_cast<const uint8_t*>(packed), static_cast<int8_t*>(out_int8), total);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda("unpack kernel launch", err);
  return 0;
}
