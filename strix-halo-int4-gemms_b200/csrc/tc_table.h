// The list of tensor-core kernel instantiations the library holds, and the record the host code keeps per
// instantiation.  The kernels are compiled in several translation units (tc_kernels.cu, once per part of the
// list) so that the library builds in parallel; the host code (b200_int4_gemms.cu) sees them only through
// these records and launches them by function pointer.
#pragma once

#include <vector>

#include "gemm_kernel.cuh"

namespace b200 {

struct TcKernelInfo {
  // what the instantiation computes
  bool int4, a_mn, b_mn;
  int scale, epi, out;
  bool mask_k, pair;
  int flavor;    // FLAVOR_* of gemm_kernel.cuh
  // how to launch it
  const void* fn;
  int threads;
  int smem_bytes;
  // setmaxnreg re-balance of the instantiation (reg_pool_needed == 0: none)
  int reg_pool_needed;
  int regs_light, regs_epilogue, regs_unpack;
  int unpack_warps;
  bool unpack_raises;
};

//   int4   A-MN   B-MN   scale     epilogue    out       maskK  pair   flavour
#define B200_FOR_EACH_TC_KERNEL(X)                                       \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)       \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_PLAIN)       \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(true, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)       \
  X(true, true, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)       \
  X(true, true, true, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)        \
  X(true, true, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)       \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)        \
  X(true, true, true, SCALE_PC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)         \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)        \
  X(true, true, true, SCALE_SC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)         \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, false, false, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(true, false, false, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)      \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_PLAIN)      \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, false, false, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(true, false, false, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(false, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(false, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(false, false, false, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, false, false, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(false, false, false, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)  \
  X(false, false, false, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)     \
  X(false, false, false, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_PLAIN)     \
  X(false, false, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, false, false, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)   \
  X(false, false, false, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)  \
  /* layout TT: A [Kb, M] with B [N, Kb] */                              \
  X(true, true, false, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(true, true, false, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_PLAIN)       \
  X(true, true, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(false, true, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(false, true, false, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  /* CTA pairs (cta_group::2): 256 x 256 output tiles over two SMs */   \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)       \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_PLAIN)      \
  X(true, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_PLAIN)     \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, true, FLAVOR_PLAIN)        \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, true, FLAVOR_PLAIN)        \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)       \
  X(true, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_PLAIN)     \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, false, true, FLAVOR_PLAIN)        \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_PLAIN)     \
  X(false, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_PLAIN)    \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, true, FLAVOR_PLAIN)       \
  X(false, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)      \
  X(false, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_PLAIN)     \
  X(false, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_PLAIN)    \
  X(false, false, false, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)     \
  X(false, false, false, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_PLAIN)    \
  X(true, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_PLAIN)      \
  X(true, true, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_PLAIN)        \
  /* per-channel int4 CTA pairs on 256 x 512 tiles */ \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_WIDE)        \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_WIDE)       \
  /* a transposed A ([K, M]) with fused activations and with subchannel scales for int8 */ \
  X(true, true, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(true, true, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, true, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(true, true, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(true, true, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC)   \
  X(true, true, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(false, true, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(false, true, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, true, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_PLAIN)      \
  X(false, true, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_PLAIN)     \
  X(false, true, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_PLAIN)    \
  X(false, true, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)   \
  X(false, true, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(false, true, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC) \
  /* grouped backward with a K-major rhs [G, N, K/2] (layouts NT, TT): bytes past a group's length are masked */ \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)        \
  X(true, true, false, SCALE_SC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)         \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)         \
  X(true, true, false, SCALE_SC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)          \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)        \
  X(true, true, false, SCALE_PC, EPI_NONE, OUT_F32, true, false, FLAVOR_PLAIN)         \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)         \
  X(true, true, false, SCALE_PC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)          \
  /* grouped backward on CTA pairs */                                    \
  X(true, true, true, SCALE_PC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)          \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)         \
  X(true, true, true, SCALE_SC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)          \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, true, true, FLAVOR_PLAIN)      \
  /* subchannel kernels in the fused accumulation order (the default of dense launches) */ \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)    \
  X(true, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC)   \
  X(true, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, false, false, FLAVOR_FUSED_SC)     \
  X(true, true, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)     \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)   \
  X(true, false, false, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(true, false, false, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC) \
  X(true, false, false, SCALE_SC, EPI_NONE, OUT_F32, false, false, FLAVOR_FUSED_SC)    \
  X(false, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)   \
  X(false, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(false, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC) \
  X(false, false, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)  \
  X(false, false, false, SCALE_SC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_FUSED_SC) \
  X(false, false, false, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_FUSED_SC) \
  X(true, true, false, SCALE_SC, EPI_NONE, OUT_BF16, false, false, FLAVOR_FUSED_SC)    \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, true, FLAVOR_FUSED_SC)     \
  X(true, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_FUSED_SC)    \
  X(true, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_FUSED_SC)   \
  X(true, false, true, SCALE_SC, EPI_NONE, OUT_F32, false, true, FLAVOR_FUSED_SC)      \
  X(false, false, true, SCALE_SC, EPI_NONE, OUT_BF16, false, true, FLAVOR_FUSED_SC)    \
  X(false, false, true, SCALE_SC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_FUSED_SC)   \
  X(false, false, true, SCALE_SC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_FUSED_SC) \
  /* per-channel int4 CTA-pair kernels with the A operand in TMEM (the default where they exist) */ \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_TMEM_A)    \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_TMEM_A)   \
  X(true, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_TMEM_A)  \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, true, FLAVOR_TMEM_A)     \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, true, FLAVOR_TMEM_A)     \
  X(true, false, false, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_TMEM_A)   \
  /* dense per-channel kernels with the balanced tail compiled in */                \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_TAIL)     \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_TAIL)    \
  X(true, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, false, FLAVOR_TAIL)   \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, false, FLAVOR_TAIL)      \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_TAIL)      \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_TAIL)      \
  X(true, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_TAIL)     \
  X(true, false, true, SCALE_PC, EPI_SWIGLU, OUT_BF16, false, true, FLAVOR_TAIL)    \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_F32, false, true, FLAVOR_TAIL)       \
  X(true, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, true, FLAVOR_TAIL)       \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, false, FLAVOR_TAIL)    \
  X(false, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, false, FLAVOR_TAIL)   \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, false, FLAVOR_TAIL)     \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_BF16, false, true, FLAVOR_TAIL)     \
  X(false, false, true, SCALE_PC, EPI_RELU2, OUT_BF16, false, true, FLAVOR_TAIL)    \
  X(false, false, true, SCALE_PC, EPI_NONE, OUT_S32, false, true, FLAVOR_TAIL)

constexpr int kTcParts = 8;  // translation units the list above is spread over (entry i goes to part i % kTcParts)

// One per part; each appends the records of the kernels compiled in its translation unit.
void tc_register_part_0(std::vector<TcKernelInfo>& out);
void tc_register_part_1(std::vector<TcKernelInfo>& out);
void tc_register_part_2(std::vector<TcKernelInfo>& out);
void tc_register_part_3(std::vector<TcKernelInfo>& out);
void tc_register_part_4(std::vector<TcKernelInfo>& out);
void tc_register_part_5(std::vector<TcKernelInfo>& out);
void tc_register_part_6(std::vector<TcKernelInfo>& out);
void tc_register_part_7(std::vector<TcKernelInfo>& out);

}  // namespace b200
