// Producers that sit either side of the GEMM path (all HBM-bound byte work, plain CUDA):
//   quantize_kernel          bf16 -> signed 4-bit codes packed along the last axis, or int8 codes
//   repack_tokens_kernel     int4 packed along features [rows, cols/2] -> packed along tokens [rows/2, cols]
//   group_info_kernel        group sizes -> row-block task arrays of the grouped forward pass
//   group_starts_kernel      group sizes -> exclusive prefix sums (first token of every group)
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

// clamp(rint(float(x) / scale), qmin, qmax): the quotient is an IEEE fp32 division and the rounding is
// round-half-to-even, as torch.round(x.float() / scale) computes it.
__device__ __forceinline__ int quantize_code(__nv_bfloat16 x, float scale, int qmin, int qmax) {
  const float q = rintf(__fdiv_rn(__bfloat162float(x), scale));
  // NaN compares false both ways and would pass through a min/max chain; torch's cast of NaN to int8 is 0
  if (!(q == q)) return 0;
  return static_cast<int>(fminf(fmaxf(q, static_cast<float>(qmin)), static_cast<float>(qmax)));
}

// One thread per 8 source values of a row (16 bytes of bf16 in, 4 bytes of int4 or 8 bytes of int8 out).
// Rows are independent; an odd `cols` pads the last byte's high nibble with a zero code.
__global__ void quantize_kernel(const __nv_bfloat16* __restrict__ src, uint8_t* __restrict__ dst,
                                long long rows, long long cols, int bits, float scale) {
  const int qmin = bits == 4 ? -8 : -128, qmax = bits == 4 ? 7 : 127;
  const long long chunks_per_row = (cols + 7) / 8;
  const long long total = rows * chunks_per_row;
  const long long dst_pitch = bits == 4 ? (cols + 1) / 2 : cols;
  const bool vector_ok = (cols % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15u) == 0);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / chunks_per_row;
    const long long c0 = (i - r * chunks_per_row) * 8;
    int code[8];
    if (vector_ok) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + r * cols + c0);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        code[2 * j] = quantize_code(__ushort_as_bfloat16(static_cast<unsigned short>(w[j] & 0xFFFFu)), scale, qmin, qmax);
        code[2 * j + 1] = quantize_code(__ushort_as_bfloat16(static_cast<unsigned short>(w[j] >> 16)), scale, qmin, qmax);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) code[j] = (c0 + j < cols) ? quantize_code(src[r * cols + c0 + j], scale, qmin, qmax) : 0;
    }
    if (bits == 4) {
      uint8_t* out = dst + r * dst_pitch + c0 / 2;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + 2 * j < cols) out[j] = static_cast<uint8_t>((code[2 * j] & 0xF) | ((code[2 * j + 1] & 0xF) << 4));
    } else {
      int8_t* out = reinterpret_cast<int8_t*>(dst) + r * dst_pitch + c0;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + j < cols) out[j] = static_cast<int8_t>(code[j]);
    }
  }
}

// Token repack for the grouped backward pass.  Source: codes of token t, feature f in nibble (f & 1) of
// src[t][f / 2].  Destination: the same code in nibble (t & 1) of dst[t / 2][f].  One thread takes two
// tokens x 8 features: 4 + 4 source bytes -> 8 destination bytes.  `cols` (features) must be even; an odd
// number of rows leaves zero codes in the high nibbles of the last destination row.
__global__ void repack_tokens_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                     long long rows, long long cols) {
  const long long src_pitch = cols / 2;
  const long long pairs = (rows + 1) / 2;
  const long long chunks_per_row = (cols + 7) / 8;
  const long long total = pairs * chunks_per_row;
  const bool vector_ok = (cols % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 3u) == 0) &&
                         ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long p = i / chunks_per_row;
    const long long f0 = (i - p * chunks_per_row) * 8;
    const bool has_odd = 2 * p + 1 < rows;
    if (vector_ok) {
      const uint32_t even = *reinterpret_cast<const uint32_t*>(src + (2 * p) * src_pitch + f0 / 2);
      const uint32_t odd = has_odd ? *reinterpret_cast<const uint32_t*>(src + (2 * p + 1) * src_pitch + f0 / 2) : 0u;
      // per source byte k (features 2k, 2k+1): low nibbles -> destination byte 2k, high nibbles -> byte 2k+1
      const uint32_t lo = (even & 0x0F0F0F0Fu) | ((odd & 0x0F0F0F0Fu) << 4);  // features 0, 2, 4, 6
      const uint32_t hi = ((even >> 4) & 0x0F0F0F0Fu) | (odd & 0xF0F0F0F0u);  // features 1, 3, 5, 7
      uint2 out;
      out.x = __byte_perm(lo, hi, 0x5140);  // f0, f1, f2, f3
      out.y = __byte_perm(lo, hi, 0x7362);  // f4, f5, f6, f7
      *reinterpret_cast<uint2*>(dst + p * cols + f0) = out;
    } else {
      for (int j = 0; j < 8; ++j) {
        const long long f = f0 + j;
        if (f >= cols) break;
        const uint8_t e = src[(2 * p) * src_pitch + f / 2];
        const uint8_t o = has_odd ? src[(2 * p + 1) * src_pitch + f / 2] : 0;
        const int sh = (f & 1) ? 4 : 0;
        dst[p * cols + f] = static_cast<uint8_t>(((e >> sh) & 0xF) | (((o >> sh) & 0xF) << 4));
      }
    }
  }
}

// Second pass of a split-K GEMM: adds the slices' partial results in ascending slice order, one thread per
// four consecutive output columns (n a multiple of 4) or per single column.
//   integer partials (per-channel scales): out = (f32(sum of s32 partials) * a_scale[row]) * b_scale[col]; the
//     integer sum is exact, so the result equals the single-pass kernel's bit for bit;
//   float partials (subchannel scales, already scaled per K-group inside each slice): out = ((p0 + p1) + p2) ...
// Deterministic either way: no atomics, a fixed order.
__global__ void splitk_reduce_kernel(const void* __restrict__ partials, float* __restrict__ out,
                                     const __nv_bfloat16* __restrict__ a_scale,
                                     const __nv_bfloat16* __restrict__ b_scale, long long rows, long long cols,
                                     int slices, int integer_partials) {
  const long long plane = rows * cols;
  const bool vec = (cols % 4) == 0;
  const long long items = vec ? plane / 4 : plane;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < items; i += stride) {
    const long long e = vec ? 4 * i : i;
    const long long row = e / cols;
    const long long col = e - row * cols;
    const int width = vec ? 4 : 1;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (integer_partials) {
      int acc[4] = {0, 0, 0, 0};
      const int* src = static_cast<const int*>(partials);
      for (int s = 0; s < slices; ++s) {
        if (vec) {
          const int4 x = *reinterpret_cast<const int4*>(src + s * plane + e);
          acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
        } else {
          acc[0] += src[s * plane + e];
        }
      }
      const float sa = __bfloat162float(a_scale[row]);
      for (int j = 0; j < width; ++j)
        v[j] = __fmul_rn(__fmul_rn(static_cast<float>(acc[j]), sa), __bfloat162float(b_scale[col + j]));
    } else {
      const float* src = static_cast<const float*>(partials);
      for (int s = 0; s < slices; ++s) {
        if (vec) {
          const float4 x = *reinterpret_cast<const float4*>(src + s * plane + e);
          v[0] = __fadd_rn(v[0], x.x); v[1] = __fadd_rn(v[1], x.y); v[2] = __fadd_rn(v[2], x.z); v[3] = __fadd_rn(v[3], x.w);
        } else {
          v[0] = __fadd_rn(v[0], src[s * plane + e]);
        }
      }
    }
    if (vec) *reinterpret_cast<float4*>(out + e) = make_float4(v[0], v[1], v[2], v[3]);
    else out[e] = v[0];
  }
}

// Exclusive prefix sums of the group sizes: starts[g] = first token of group g, starts[groups] = total.
// One CTA of 1024 threads; groups are scanned in slabs of 1024 with a running carry.
__global__ void group_starts_kernel(const long long* __restrict__ sizes, long long* __restrict__ starts,
                                    int groups) {
  __shared__ long long slab[1024];
  __shared__ long long carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < groups; base += 1024) {
    const int g = base + threadIdx.x;
    const long long mine = g < groups ? max(sizes[g], 0ll) : 0;
    slab[threadIdx.x] = mine;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {  // Hillis-Steele inclusive scan
      const long long add = threadIdx.x >= off ? slab[threadIdx.x - off] : 0;
      __syncthreads();
      slab[threadIdx.x] += add;
      __syncthreads();
    }
    if (g < groups) starts[g] = carry + slab[threadIdx.x] - mine;
    __syncthreads();
    if (threadIdx.x == 1023) carry += slab[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) starts[groups] = carry;
}

// Row-block tasks of the grouped forward pass, built on the device so that the task count never has to
// travel to the host.  For group g with rows [s, e): aligned = floor(s / align) * align; blocks of `tile`
// rows from `aligned` cover [s, e); task b of the group: block_start = aligned + b * tile,
// actual_start = max(block_start, s), actual_end = min(block_start + tile, e).  Empty groups make no
// task.  Tasks are written in group order; entries from *num_tasks to max_tasks are zero-size tasks
// (group 0, all bounds 0).  One CTA of 1024 threads.
__global__ void group_info_kernel(const long long* __restrict__ sizes, int groups, int tile, int align,
                                  long long* __restrict__ task_group, long long* __restrict__ task_block_start,
                                  long long* __restrict__ task_actual_start, long long* __restrict__ task_actual_end,
                                  int max_tasks, int* __restrict__ num_tasks, int* __restrict__ overflow) {
  __shared__ long long slab_rows[1024];
  __shared__ int slab_tasks[1024];
  __shared__ long long carry_rows;
  __shared__ int carry_tasks;
  if (threadIdx.x == 0) {
    carry_rows = 0;
    carry_tasks = 0;
  }
  __syncthreads();
  for (int base = 0; base < groups; base += 1024) {
    const int g = base + threadIdx.x;
    const long long size = g < groups ? max(sizes[g], 0ll) : 0;  // negative sizes count as empty (reference ragged.py:244)
    slab_rows[threadIdx.x] = size;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const long long add = threadIdx.x >= off ? slab_rows[threadIdx.x - off] : 0;
      __syncthreads();
      slab_rows[threadIdx.x] += add;
      __syncthreads();
    }
    const long long start = carry_rows + slab_rows[threadIdx.x] - size;
    const long long end = start + size;
    const long long aligned = (start / align) * align;
    const int blocks = size > 0 ? static_cast<int>((end - aligned + tile - 1) / tile) : 0;
    slab_tasks[threadIdx.x] = blocks;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int add = threadIdx.x >= off ? slab_tasks[threadIdx.x - off] : 0;
      __syncthreads();
      slab_tasks[threadIdx.x] += add;
      __syncthreads();
    }
    const int first = carry_tasks + slab_tasks[threadIdx.x] - blocks;
    for (int b = 0; b < blocks; ++b) {
      const int t = first + b;
      if (t >= max_tasks) break;
      const long long bs = aligned + static_cast<long long>(b) * tile;
      task_group[t] = g;
      task_block_start[t] = bs;
      task_actual_start[t] = bs > start ? bs : start;
      task_actual_end[t] = bs + tile < end ? bs + tile : end;
    }
    __syncthreads();
    if (threadIdx.x == 1023) {
      carry_rows += slab_rows[1023];
      carry_tasks += slab_tasks[1023];
    }
    __syncthreads();
  }
  const int total = carry_tasks;
  for (int t = total + threadIdx.x; t < max_tasks; t += blockDim.x) {
    task_group[t] = 0;
    task_block_start[t] = 0;
    task_actual_start[t] = 0;
    task_actual_end[t] = 0;
  }
  if (threadIdx.x == 0) {
    *num_tasks = total < max_tasks ? total : max_tasks;
    *overflow = total > max_tasks ? 1 : 0;
  }
}

}  // namespace b200
