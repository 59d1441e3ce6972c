// CUDA-core GEMM for the shapes the tensor-core kernel does not take (operand pitches
// that are not multiples of 16 bytes, K-major B, tiny problems).  Same math, same operand
// format, any layout, any K including odd K; one thread per output element, exact int32
// accumulation per K-group.  It is a device kernel like the others: there is no host
// fallback anywhere in the library.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

#include "gemm_kernel.cuh"

namespace b200 {

struct SimtParams {
  int mode;            // MODE_*
  int int4;            // 1: packed nibbles, 0: int8
  int a_transposed;    // A stored [Kb, M]
  int b_transposed;    // B stored [N, Kb]
  int scale_mode;      // SCALE_*
  int subchannel;
  int scale_cols;
  int epilogue;
  int out_dtype;
  int M, N, K;         // logical; N = output columns (SwiGLU: D)
  int b_cols;          // stored B columns (SwiGLU: 2*D)
  int kb;              // K bytes per row/column of an operand (pitch of the K-major forms)
  int num_groups;
  int num_tasks;
  const uint8_t* a;
  const uint8_t* b;
  const __nv_bfloat16* a_scale;
  const __nv_bfloat16* b_scale;
  const long long* task_group_ids;
  const long long* task_actual_starts;
  const long long* task_actual_ends;
  const long long* group_sizes;
  const long long* group_starts;  // bwd, flat token-packed operands (see GemmParams::group_starts); else nullptr
  void* out;
};

__device__ __forceinline__ int load_q(const uint8_t* base, long long byte_index, int k, int int4) {
  const uint8_t v = base[byte_index];
  if (!int4) return static_cast<int>(static_cast<int8_t>(v));
  const int nib = (k & 1) ? (v >> 4) : (v & 0xF);
  return (nib >= 8) ? nib - 16 : nib;
}

// grid: x over columns (64 per block), y over rows (4 per block) ; z over groups (bwd) or tasks (fwd)
__global__ void gemm_simt_kernel(const SimtParams p) {
  const int col = blockIdx.x * 64 + (threadIdx.x & 63);
  int row = blockIdx.y * 4 + (threadIdx.x >> 6);
  if (col >= p.N) return;

  int g = 0;
  int k_len = p.K;
  long long k_base = 0;  // flat backward operands: token index of the group's k = 0
  long long a_group_off = 0, b_group_off = 0, out_off = 0, sa_off = 0, sb_off = 0;
  const int sc = (p.scale_mode == SCALE_SC) ? p.scale_cols : 1;
  if (p.mode == MODE_RAGGED_FWD) {
    const int task = blockIdx.z;
    const int lo = max(0, static_cast<int>(p.task_actual_starts[task]));
    const int hi = min(p.M, static_cast<int>(p.task_actual_ends[task]));
    row += lo;
    if (row >= hi) return;
    g = static_cast<int>(p.task_group_ids[task]);
    b_group_off = static_cast<long long>(g) * p.kb * p.b_cols;
    sb_off = static_cast<long long>(g) * sc * p.b_cols;
  } else if (p.mode == MODE_RAGGED_BWD) {
    g = blockIdx.z;
    if (row >= p.M) return;
    k_len = static_cast<int>(p.group_sizes[g]);
    if (p.group_starts != nullptr) {
      k_base = p.group_starts[g];
    } else {
      a_group_off = static_cast<long long>(g) * p.kb * p.M;
      b_group_off = static_cast<long long>(g) * p.kb * p.b_cols;
    }
    out_off = static_cast<long long>(g) * p.M * p.N;
    sa_off = static_cast<long long>(g) * p.M * sc;
    sb_off = static_cast<long long>(g) * sc * p.b_cols;
  } else {
    if (row >= p.M) return;
  }

  const uint8_t* a = p.a + a_group_off;
  const uint8_t* b = p.b + b_group_off;
  const int group_len = (p.scale_mode == SCALE_SC) ? p.subchannel : 0x7FFFFFFF;
  const bool swiglu = (p.epilogue == EPI_SWIGLU);

  float out_up = 0.f, out_gate = 0.f;
  int acc_up = 0, acc_gate = 0;
  int gi = 0;
  for (int k0 = 0; k0 < k_len || (k0 == 0 && p.scale_mode == SCALE_PC); k0 += group_len) {
    const int k1 = (group_len == 0x7FFFFFFF) ? k_len : min(k0 + group_len, k_len);
    acc_up = 0;
    acc_gate = 0;
    for (int k = k0; k < k1; ++k) {
      const long long kk = k_base + k;  // position along the stored K axis (differs from k for flat operands)
      const long long kbyte = p.int4 ? (kk >> 1) : kk;
      const int knib = static_cast<int>(kk & 1);
      const long long ai = p.a_transposed ? (kbyte * p.M + row) : (static_cast<long long>(row) * p.kb + kbyte);
      const int av = load_q(a, ai, knib, p.int4);
      const long long bi = p.b_transposed ? (static_cast<long long>(col) * p.kb + kbyte) : (kbyte * p.b_cols + col);
      acc_up += av * load_q(b, bi, knib, p.int4);
      if (swiglu) {
        const long long bg = p.b_transposed ? (static_cast<long long>(col + p.N) * p.kb + kbyte)
                                            : (kbyte * p.b_cols + col + p.N);
        acc_gate += av * load_q(b, bg, knib, p.int4);
      }
    }
    if (p.out_dtype == OUT_S32) break;
    if (p.scale_mode == SCALE_PC) {
      const float sa = __bfloat162float(p.a_scale[sa_off + row]);
      out_up = __fmul_rn(__fmul_rn(static_cast<float>(acc_up), sa), __bfloat162float(p.b_scale[sb_off + col]));
      if (swiglu)
        out_gate = __fmul_rn(__fmul_rn(static_cast<float>(acc_gate), sa),
                             __bfloat162float(p.b_scale[sb_off + col + p.N]));
      break;
    }
    const float sa = __bfloat162float(p.a_scale[sa_off + static_cast<long long>(row) * sc + gi]);
    const __nv_bfloat16* sb_row = p.b_scale + sb_off + static_cast<long long>(gi) * p.b_cols;
    out_up = __fadd_rn(out_up, __fmul_rn(__fmul_rn(static_cast<float>(acc_up), sa), __bfloat162float(sb_row[col])));
    if (swiglu)
      out_gate = __fadd_rn(out_gate, __fmul_rn(__fmul_rn(static_cast<float>(acc_gate), sa),
                                               __bfloat162float(sb_row[col + p.N])));
    ++gi;
  }

  const long long o = out_off + static_cast<long long>(row) * p.N + col;
  if (p.out_dtype == OUT_S32) {
    reinterpret_cast<int*>(p.out)[o] = acc_up;
    return;
  }
  float v = out_up;
  if (swiglu) {
    v = out_up * (out_gate / (1.0f + __expf(-out_gate)));
  } else if (p.epilogue == EPI_RELU2) {
    v = fmaxf(v, 0.f);
    v = v * v;
  }
  if (p.out_dtype == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p.out)[o] = v;
}

// packed int4 [rows, cols_packed] -> int8 [rows, 2*cols_packed]; 16 packed bytes per thread.
__global__ void unpack_int4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ out,
                                   long long total_bytes) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 16;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 16;
       i < total_bytes; i += stride) {
    if (i + 16 <= total_bytes) {
      const uint4 x = *reinterpret_cast<const uint4*>(packed + i);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // bytes b0..b3 -> int8 (lo0, hi0, lo1, hi1) and (lo2, hi2, lo3, hi3)
        const uint32_t lo = w[j] & 0x0F0F0F0Fu;
        const uint32_t hi = (w[j] >> 4) & 0x0F0F0F0Fu;
        // sign-extend each nibble held in a byte: v | (v & 8) * 0x1E  (8 * 0x1E = 0xF0)
        const uint32_t slo = lo | ((lo & 0x08080808u) * 0x1Eu);
        const uint32_t shi = hi | ((hi & 0x08080808u) * 0x1Eu);
        o[2 * j] = __byte_perm(slo, shi, 0x5140);      // lo0 hi0 lo1 hi1
        o[2 * j + 1] = __byte_perm(slo, shi, 0x7362);  // lo2 hi2 lo3 hi3
      }
      uint4* dst = reinterpret_cast<uint4*>(out + 2 * i);
      dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
      dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
      for (long long j = i; j < total_bytes; ++j) {
        const uint8_t v = packed[j];
        const int lo = v & 0xF, hi = v >> 4;
        out[2 * j] = static_cast<int8_t>(lo >= 8 ? lo - 16 : lo);
        out[2 * j + 1] = static_cast<int8_t>(hi >= 8 ? hi - 16 : hi);
      }
    }
  }
}

}  // namespace b200
