// Tensor-core kernel instantiations, part B200_TC_PART of kTcParts (compiled once per part, in parallel).
// Each part instantiates every kTcParts-th entry of B200_FOR_EACH_TC_KERNEL and hands the host code one
// TcKernelInfo record per kernel.
#include "tc_table.h"

#ifndef B200_TC_PART
#error "compile with -DB200_TC_PART=<0..kTcParts-1>"
#endif

namespace b200 {
namespace {

template <bool I4, bool AMN, bool BMN, int SC, int EP, int OT, bool MK, bool PR, int FL>
TcKernelInfo describe() {
  using T = KernelTraits<I4, AMN, BMN, SC, EP, OT, MK, PR, FL>;
  TcKernelInfo info{};
  info.int4 = I4;
  info.a_mn = AMN;
  info.b_mn = BMN;
  info.scale = SC;
  info.epi = EP;
  info.out = OT;
  info.mask_k = MK;
  info.pair = PR;
  info.flavor = FL;
  info.fn = reinterpret_cast<const void*>(&gemm_i8_tcgen05_kernel<I4, AMN, BMN, SC, EP, OT, MK, PR, FL>);
  info.threads = T::kThreads;
  info.smem_bytes = T::kSmemBytes;
  info.reg_pool_needed = T::kRegPoolNeeded;
  info.regs_light = T::kRegsLight;
  info.regs_epilogue = T::kRegsEpilogue;
  info.regs_unpack = T::kRegsUnpack;
  info.unpack_warps = T::kUnpackWarps;
  info.unpack_raises = T::kUnpackRaises;
  return info;
}

// The branch is discarded (and its kernel not instantiated) unless the entry's index falls in kPart: the
// condition depends on the template parameter.
template <int kPart>
void register_part(std::vector<TcKernelInfo>& out) {
  constexpr int kBase = __COUNTER__ + 1;
#define X(I4, AMN, BMN, SC, EP, OT, MK, PR, FL) \
  if constexpr ((__COUNTER__ - kBase) % kTcParts == kPart) out.push_back(describe<I4, AMN, BMN, SC, EP, OT, MK, PR, FL>());
  B200_FOR_EACH_TC_KERNEL(X)
#undef X
}

}  // namespace

#define B200_CONCAT2(a, b) a##b
#define B200_CONCAT(a, b) B200_CONCAT2(a, b)
void B200_CONCAT(tc_register_part_, B200_TC_PART)(std::vector<TcKernelInfo>& out) { register_part<B200_TC_PART>(out); }

}  // namespace b200
