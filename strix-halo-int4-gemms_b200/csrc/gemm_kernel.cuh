// Persistent, warp-specialised integer GEMM for sm_100a.
//
//   C[M,N] = epilogue( sum over K-groups( s32( A_q @ B_q ) * sA * sB ) )
//
// One CTA per SM walks a list of 128 x 256 output tiles.  Roles (warps):
//   warp 0        TMA producer: brings packed-int4 (or int8) operand tiles into shared memory
//   warp 1        MMA issuer: one thread issues tcgen05.mma kind::i8 (s8 x s8 -> s32 in TMEM)
//   warps 2..     epilogue: tcgen05.ld the accumulator, scale in fp32, activation, store
//   last 8 warps  (int4 only) unpack: expand nibbles to int8 into the swizzled UMMA tiles
//
// int4 operands.  Blackwell tensor cores have no int4 MMA, so each nibble v becomes the
// int8 value 16*v (the nibble moved to the top of its byte, no sign-extension arithmetic).
// The s32 accumulator then holds 256 * sum(a*b), exactly, and the epilogue shifts it right
// by 8 (arithmetic, exact) before converting to fp32.  |sum| <= 64*K, so this is safe for
// K < 131072, which the host side checks.
//
// K order inside a 128-wide K block.  A dot product does not care about the order of its
// terms as long as A and B use the same order.  Packed byte p of a block (p = 0..63) holds
// k = 2p (low nibble) and k = 2p+1 (high nibble).  Its low nibble goes to K slot
// 32*(p/16) + p%16 and its high nibble to that slot + 16, for both operands.  A 16-byte
// load of packed data therefore produces two whole 16-byte chunks of int8, and each K=32
// MMA step still covers one contiguous range of 32 original k indices (so K-groups of
// 32/64/128/256 keep their boundaries).
//
// Shared-memory tiles use the 128-byte-swizzle UMMA canonical layouts:
//   A, K-major  : [128 rows][128 B of K], 16-byte chunk c of row r stored at chunk c ^ (r & 7)
//   A/B MN-major: per 128-wide M/N block [128 K rows][128 B of M/N], chunk c of K row s at c ^ (s & 7)
// int8 operands are written there directly by TMA (SWIZZLE_128B), int4 by the unpack warps.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

#include "ptx.cuh"

namespace b200 {

enum : int { MODE_DENSE = 0, MODE_RAGGED_FWD = 1, MODE_RAGGED_BWD = 2 };
enum : int { SCALE_PC = 0, SCALE_SC = 1 };
enum : int { EPI_NONE = 0, EPI_RELU2 = 1, EPI_SWIGLU = 2 };
enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_S32 = 2 };

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;   // logical K per pipeline stage
constexpr int NBLK = 128; // width of one M/N block of an MN-major operand (bytes == elements)
constexpr int TMEM_COLS = 512;

struct GemmParams {
  int mode;
  int M, N, K;           // logical problem: rows, output columns (SwiGLU: D), reduction length
  int tiles_m, tiles_n;  // dense / ragged-bwd tile grid (per group for bwd)
  int num_tiles;
  int group_m;           // raster swizzle width (dense)
  int tile_cols;         // output columns per tile: 256, or 128 for SwiGLU (up + gate blocks)
  int gate_col_offset;   // column distance from the first to the second 128-wide B block:
                         // 128 normally, D (the gate half) for SwiGLU
  int ldc;               // output row pitch in elements
  int subchannel;        // K-group length for subchannel scales (0 = per-channel)
  int scale_cols;        // number of K-groups (subchannel) per row
  int lds_b;             // pitch (elements) of one b_scale K-group row
  int tma_store;         // 1: tmap_c describes the output and the epilogue may use TMA stores
  // split-K (dense): slice s reduces k in [s * k_per_slice, min(K, (s + 1) * k_per_slice)) and writes its partial
  // result to out + s * M * ldc (a [k_slices, M, N] workspace); a second kernel adds the slices in a fixed order
  int k_slices;          // 1: no split
  int k_per_slice;       // multiple of BK (and of the K-group length)
  // balanced tail (dense, per-channel).  Whole tiles go round-robin over the scheduling units (CTA pairs or CTAs) for
  // the full waves; the tail_rest tiles of the last, partly filled wave are cut along K into tail_split parts that run
  // on different units at the same time.  Part 0 is the tile's owner: it is the LAST segment of units 0 .. rest-1 and
  // starts from the sum of the other parts (exact s32 partial sums), which units p * rest + j (part p of rest tile j)
  // produce as their FIRST segment, store to tail_partials and announce in tail_flags.
  int tail_units;        // 0: off; else the number of scheduling units of the launch
  int tail_split;        // parts per rest tile (2 .. 4)
  int tail_waves;        // full waves of whole tiles
  int tail_rest;         // tiles of the last wave
  int tail_kb_per_tile;
  int* tail_partials;    // [units][2 ranks][128][256] s32
  int* tail_flags;       // [units][2 ranks][2]: epilogue warps that have written their part, and readers that have seen
                         // it; zero before the first launch on a workspace, and again at the end of every launch
  // wide kernels, dense: mixed column cuts.  The first mix_rows_hi row tiles hold mix_wide_hi tiles of 512 columns
  // followed by mix_tq_hi tiles of 384, the other row tiles mix_wide_lo and mix_tq_lo; the tile list has all the
  // 512-column tiles first (mix_total_wide of them) and then the 384-column ones, so that the last wave of the
  // round-robin schedule holds tiles of three quarters of the width only.  mix_total_wide < 0: one width (tile_cols)
  int mix_total_wide, mix_rows_hi, mix_wide_hi, mix_wide_lo, mix_tq_hi, mix_tq_lo;
  // ragged
  int num_groups;
  int rows_per_group_a;  // rows of the stacked A map per group (bwd)
  int rows_per_group_b;  // rows of the stacked B map per group (packed K rows for int4)
  const long long* task_group_ids;
  const long long* task_block_starts;
  const long long* task_actual_starts;
  const long long* task_actual_ends;
  const long long* group_sizes;  // bwd: valid K per group
  // bwd, flat operands: lhs [ceil(rows/2), M] and rhs [ceil(rows/2), N] hold all tokens back to back,
  // packed in pairs along the token axis; group g reduces over tokens [group_starts[g], +group_sizes[g]).
  // nullptr: operands are stacked per group and padded to a common capacity.
  const long long* group_starts;
  const int* num_tasks_dev;      // fwd: task count left on the device by the task builder (nullptr: tiles_m)
  const int* overflow_dev;       // fwd: the builder's "tasks did not fit" flag (nullptr: not checked)
  const __nv_bfloat16* a_scale;
  const __nv_bfloat16* b_scale;
  void* out;
  int* status;  // host-mapped int[4] or nullptr
};

struct TileWork {
  int a_x, a_y;      // TMA coordinates of the first A box of the tile (K block 0)
  int b_y;           // TMA row coordinate of the first B box
  int n0, n1;        // column origins of the two 128-wide B blocks
  int kb0;           // first K block (split-K slices start past 0)
  int num_kb;        // K blocks to run
  int k_len;         // reduction length of this tile (bwd: group_sizes[g])
  int k_valid;       // number of valid k (masking, bwd); INT_MAX otherwise
  int k_first;       // first valid k (1 when a flat group starts on the odd token of a byte, else 0)
  int part;          // balanced tail: PART_WHOLE, PART_OWNER (part 0 + the other parts' partial sums), PART_PRODUCER
  int part_slot;     // partial-sum slot written (producer: its own unit)
  int tq;            // wide kernels: 1 = the tile is 384 columns wide (its second MMA has N = 128: 64 columns per CTA)
  int out_row0;      // output row of tile row 0
  int row_lo, row_hi;// valid output rows [lo, hi)
  long long out_off; // element offset added to out (bwd: g*M*N)
  int out_row_base;  // row offset of the tile's output in the 2-D view [rows, N] (bwd: g*M)
  long long sa_off;  // element offset of this tile's a_scale base
  long long sb_off;  // element offset of this tile's b_scale base
};

enum : int { PART_WHOLE = 0, PART_OWNER = 1, PART_PRODUCER = 2 };

// `rank` is the CTA's rank in its pair (always 0 for single-CTA kernels); `unit` the scheduling unit (cluster or CTA)
// index, used by the balanced-tail schedule, in which `t` counts the unit's own segments.  A pair works on 256 rows of
// output: rank r owns rows [128 r, 128 r + 128) of them, and p.tiles_m counts 256-row tiles.
template <bool kAMn, bool k2Cta, bool kTail = false, bool kWide = false>
__device__ __forceinline__ TileWork decode_tile(const GemmParams& p, int t, int rank, int unit) {
  constexpr int RM = k2Cta ? 2 * BM : BM;  // output rows per scheduled tile
  const int rank_rows = k2Cta ? rank * BM : 0;
  TileWork w;
  w.k_valid = 0x7FFFFFFF;
  w.k_first = 0;
  w.kb0 = 0;
  w.part = PART_WHOLE;
  w.part_slot = 0;
  w.tq = 0;
  w.out_off = 0;
  w.out_row_base = 0;
  w.sa_off = 0;
  w.sb_off = 0;
  if (p.mode == MODE_DENSE) {
    // balanced tail: segment t of this unit (a producer part first, whole tiles, an owner part last)
    int seg_kb0 = 0, seg_kb1 = 0;
    if (kTail && p.tail_units > 0) {
      const int kbt = p.tail_kb_per_tile;
      const bool producer = unit >= p.tail_rest && unit < p.tail_split * p.tail_rest;
      const int wave = producer ? t - 1 : t;
      seg_kb1 = kbt;
      if (wave >= 0 && wave < p.tail_waves) {
        t = wave * p.tail_units + unit;
      } else {
        const int part = producer ? unit / p.tail_rest : 0;
        t = p.tail_waves * p.tail_units + unit % p.tail_rest;
        seg_kb0 = part * kbt / p.tail_split;
        seg_kb1 = (part + 1) * kbt / p.tail_split;
        w.part = producer ? PART_PRODUCER : PART_OWNER;
        w.part_slot = unit;
      }
    }
    // split-K: the slice is the slowest index of the tile list
    int slice = 0;
    if (p.k_slices > 1) {
      const int per_slice = p.tiles_m * p.tiles_n;
      slice = t / per_slice;
      t -= slice * per_slice;
    }
    // grouped raster: walk group_m row-tiles down before moving to the next column tile
    const int per_group = p.group_m * p.tiles_n;
    const int grp = t / per_group;
    const int first_m = grp * p.group_m;
    const int rows_here = min(p.tiles_m - first_m, p.group_m);
    const int local = t - grp * per_group;
    int mt = first_m + local % rows_here;
    const int nt = local / rows_here;
    int n0 = nt * p.tile_cols;
    if (kWide && p.mix_total_wide >= 0) {
      // mixed column cuts: row by row, the 512-column tiles of every row first, then the 384-column ones
      const bool tq = t >= p.mix_total_wide;
      const int u = tq ? t - p.mix_total_wide : t;
      const int per_hi = tq ? p.mix_tq_hi : p.mix_wide_hi, per_lo = tq ? p.mix_tq_lo : p.mix_wide_lo;
      const int hi_span = p.mix_rows_hi * per_hi;
      int idx;
      if (u < hi_span) {
        mt = u / per_hi;
        idx = u - mt * per_hi;
      } else {
        const int r = (u - hi_span) / per_lo;
        mt = p.mix_rows_hi + r;
        idx = (u - hi_span) - r * per_lo;
      }
      const int wide_before = tq ? (mt < p.mix_rows_hi ? p.mix_wide_hi : p.mix_wide_lo) : 0;
      n0 = wide_before * (2 * BN) + idx * (tq ? 3 * NBLK : 2 * BN);
      w.tq = tq ? 1 : 0;
    }
    w.a_x = kAMn ? mt * RM + rank_rows : 0;
    w.a_y = kAMn ? 0 : mt * RM + rank_rows;
    w.b_y = 0;
    w.n0 = n0;
    w.n1 = w.n0 + p.gate_col_offset;
    w.k_len = p.K;
    if (p.k_slices > 1) {
      const int k0 = slice * p.k_per_slice;
      w.kb0 = k0 / BK;
      w.k_len = max(0, min(p.K - k0, p.k_per_slice));
      w.out_off = static_cast<long long>(slice) * p.M * p.ldc;
      w.out_row_base = slice * p.M;
      if (p.subchannel) {
        const int groups_per_slice = p.k_per_slice / p.subchannel;
        w.sa_off = static_cast<long long>(slice) * groups_per_slice;
        w.sb_off = static_cast<long long>(slice) * groups_per_slice * p.lds_b;
      }
    }
    if (kTail && p.tail_units > 0) {
      w.kb0 = seg_kb0;
      w.k_len = min(p.K, seg_kb1 * BK) - seg_kb0 * BK;
    }
    w.num_kb = (w.k_len + BK - 1) / BK;
    w.out_row0 = mt * RM + rank_rows;
    w.row_lo = w.out_row0;
    w.row_hi = min(p.M, w.out_row0 + BM);
  } else if (p.mode == MODE_RAGGED_FWD) {
    const int task = t / p.tiles_n;
    const int nt = t - task * p.tiles_n;
    const int g = static_cast<int>(p.task_group_ids[task]);
    const int bs = static_cast<int>(p.task_block_starts[task]);
    // a transposed lhs [K/2, M] has the task's rows on the TMA x axis
    w.a_x = kAMn ? bs + rank_rows : 0;
    w.a_y = kAMn ? 0 : bs + rank_rows;
    w.b_y = g * p.rows_per_group_b;
    w.n0 = nt * p.tile_cols;  // 256, or 512 for the wide kernels
    w.n1 = w.n0 + NBLK;
    w.k_len = p.K;
    w.num_kb = (p.K + BK - 1) / BK;
    w.out_row0 = bs + rank_rows;
    // task bounds come from the caller (or from the device-side builder): never trust them past the operand
    w.row_lo = max(0, static_cast<int>(p.task_actual_starts[task]));
    w.row_hi = min(p.M, static_cast<int>(p.task_actual_ends[task]));
    if (kAMn && (bs & 15) != 0) {
      // an x coordinate that is not a multiple of 16 bytes must never reach TMA: every role skips the task (no K
      // blocks, no rows), and the CTA that meets it first says so in the status word
      w.num_kb = 0;
      w.row_hi = w.row_lo;
      if (p.status != nullptr && threadIdx.x == 0 && p.status[0] == STATUS_OK) {
        p.status[1] = task;
        p.status[2] = 0;
        p.status[0] = STATUS_TASK_ALIGNMENT;
      }
    }
    w.sb_off = static_cast<long long>(g) * p.lds_b * (p.subchannel ? p.scale_cols : 1);
  } else {
    const int per_g = p.tiles_m * p.tiles_n;
    const int g = t / per_g;
    const int local = t - g * per_g;
    const int mt = local / p.tiles_n;
    const int nt = local - mt * p.tiles_n;
    int kg = static_cast<int>(p.group_sizes[g]);
    w.a_x = kAMn ? mt * RM + rank_rows : 0;
    if (p.group_starts != nullptr) {
      // flat operands (token-major lhs only): the group's first byte row, and one leading nibble to
      // skip when the group starts on an odd token; an empty group stays empty
      const long long start = p.group_starts[g];
      w.k_first = kg > 0 ? static_cast<int>(start & 1) : 0;
      kg += w.k_first;
      w.a_y = static_cast<int>(start >> 1);
      w.b_y = w.a_y;
    } else {
      w.a_y = kAMn ? g * p.rows_per_group_a : g * p.rows_per_group_a + mt * RM + rank_rows;
      w.b_y = g * p.rows_per_group_b;
    }
    w.n0 = nt * BN;
    w.n1 = w.n0 + NBLK;
    w.k_valid = kg;
    w.k_len = kg;
    w.num_kb = (kg + BK - 1) / BK;
    w.out_row0 = mt * RM + rank_rows;
    w.row_lo = w.out_row0;
    w.row_hi = min(p.M, w.out_row0 + BM);
    w.out_off = static_cast<long long>(g) * p.M * p.ldc;
    w.out_row_base = g * p.M;
    w.sa_off = static_cast<long long>(g) * p.M * (p.subchannel ? p.scale_cols : 1);
    w.sb_off = static_cast<long long>(g) * p.lds_b * (p.subchannel ? p.scale_cols : 1);
  }
  // wide kernels: a last column tile that holds between 257 and 384 columns runs as a 384-column tile as well
  if (kWide && p.N - w.n0 <= 3 * NBLK && p.N - w.n0 > 2 * NBLK) w.tq = 1;
  return w;
}

// Expand four packed bytes (8 nibbles) into two words of int8 = 16 * nibble value.
__device__ __forceinline__ void expand_word(uint32_t w, uint32_t& lo, uint32_t& hi) {
  lo = (w << 4) & 0xF0F0F0F0u;
  hi = w & 0xF0F0F0F0u;
}

// Balanced tail: adds the other parts' partial sums (chunks [c_begin, c_end) of 32 columns, this thread's row) into the
// accumulator buffer at `acc` (TMEM address of the warp's lanes, column 0 of the buffer).  `keep_own`: the buffer
// already holds this unit's own sum (added to), else it is overwritten.  Slot layout: 16-byte piece i of chunk c of
// row r at int4 index ((c * 8 + i) * 128 + r), so that a warp's 32 rows move 512 contiguous bytes per instruction.
// Kept out of line: it runs once per launch and unit, and its registers must not weigh on the epilogue proper.
static __device__ __noinline__ void tail_sum_into_tmem(uint32_t acc, const int4* first_part, long long part_stride, int parts,
                                                int c_begin, int c_end, bool keep_own) {
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t r[32];
    if (keep_own) {
      tmem_ld_32x32b_x32(acc + 32 * c, r);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0u;
    }
    for (int part = 0; part < parts; ++part) {
      const int4* src = first_part + part * part_stride;
      int4 x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = __ldcg(src + (c * 8 + i) * BM);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        r[4 * i] += static_cast<uint32_t>(x[i].x);
        r[4 * i + 1] += static_cast<uint32_t>(x[i].y);
        r[4 * i + 2] += static_cast<uint32_t>(x[i].z);
        r[4 * i + 3] += static_cast<uint32_t>(x[i].w);
      }
    }
    tmem_st_32x32b_x32(acc + 32 * c, r);
  }
  tmem_st_wait();
}

// Kernel flavours (mutually exclusive refinements of an instantiation):
//   FLAVOR_FUSED_SC  subchannel kernels: the fused order of roundings of the per-K-group accumulation (see the kernel)
//   FLAVOR_TMEM_A    per-channel int4 CTA-pair kernels with a row-major A: the unpacked A operand goes to TMEM
//                    (tcgen05.st by the unpack warps, tcgen05.mma with a TMEM A operand) instead of shared memory
//   FLAVOR_TAIL      per-channel kernels that can run the balanced tail (GemmParams::tail_units): the code for parts of
//                    tiles and their partial sums is compiled into these instantiations only, so that it does not
//                    weigh on the register allocation of the plain kernels
//   FLAVOR_WIDE      per-channel int4 CTA-pair kernels with tiles of 256 x 512: every CTA unpacks its 128 rows of A once
//                    per K block for TWO 128-column blocks of B (two MMAs of N = 256 per K step), a quarter less
//                    unpack work and shared-memory traffic per output element; the 512 TMEM columns hold one
//                    accumulator, so a tile's epilogue (eight warps) is not hidden behind the next tile's MMAs.
//                    Two int8 stages and four packed ones: what counts is how far ahead TMA runs (measured at
//                    4096^3: 54.6 us with 3 + 2 stages, 52.8 with 2 + 3, 52.1 with 2 + 4)
enum : int { FLAVOR_PLAIN = 0, FLAVOR_FUSED_SC = 1, FLAVOR_TMEM_A = 2, FLAVOR_TAIL = 3, FLAVOR_WIDE = 5 };

template <bool kInt4, bool kAMn, bool kBMn, int kScale, int kEpi, int kOut, bool kMaskK, bool k2Cta = false, int kFlavor = FLAVOR_PLAIN>
struct KernelTraits {
  static constexpr bool kFastSc = kFlavor == FLAVOR_FUSED_SC;
  // A through TMEM.  The int4 kernels are bound by the shared-memory data pipe: per 128-deep K block a CTA of a
  // pair writes 16 KB of unpacked A to shared memory and the tensor core reads it back.  With A in TMEM neither
  // crosses that pipe (a third of its traffic).  TMEM then holds ONE 256-column accumulator (the epilogue of a
  // tile no longer overlaps the next tile's MMAs) and seven 32-column A stages; the deeper operand pipeline
  // (seven stages filled during the epilogue) wins most of that overlap back.
  static constexpr bool kTmemA = kFlavor == FLAVOR_TMEM_A;
  static_assert(!kTmemA || (kInt4 && !kAMn && k2Cta && kScale == SCALE_PC && !kMaskK),
                "A through TMEM: per-channel int4 CTA-pair kernels with a row-major A");
  static constexpr bool kTail = kFlavor == FLAVOR_TAIL;
  static_assert(!kTail || (kScale == SCALE_PC && !kMaskK), "the balanced tail belongs to the dense per-channel kernels");
  static constexpr bool kWide = kFlavor == FLAVOR_WIDE;
  static_assert(!kWide || (kInt4 && !kAMn && kBMn && k2Cta && kScale == SCALE_PC && !kMaskK && kEpi != EPI_SWIGLU && kOut == OUT_BF16),
                "wide tiles: per-channel int4 CTA-pair kernels, NN layout, bf16 output, no gate block");
  static constexpr int kAccBufs = (kTmemA || kWide) ? 1 : 2;  // accumulator buffers (256 TMEM columns; wide: one of 512)
  static constexpr int kTmemAStage0 = 256;                 // first TMEM column of the A stages (32 columns each)
  // Eight unpack warps beside the eight epilogue warps of a subchannel kernel were tried (640 threads: 168 registers
  // for the epilogue, 56 for the unpack warps): the spills made it a third slower than four unpack warps.
  static constexpr bool kWideSc = false;
  // K-masked kernels serve the grouped backward pass: short reductions (a group's tokens) and large fp32
  // tiles.  Their epilogue is the long pole, so it gets eight warps (two per TMEM lane quarter, half of the
  // columns each) and one of the operand stages as output staging.
  static constexpr bool kShortK = kMaskK && kInt4;
  // Kernels with eight epilogue warps re-balance registers between roles with setmaxnreg, which works on
  // warpgroups (4 consecutive warps): warps 0..3 = TMA, MMA and two idle warps, 4..11 = epilogue, then unpack
  // (4 warps next to the subchannel epilogue, whose running sums need 200 registers; 8 warps otherwise).
  static constexpr bool kRegBalance = (kScale == SCALE_SC) || kShortK || kTmemA || kWide;
  static constexpr int kUnpackWarps = kInt4 ? ((kScale == SCALE_SC && !kWideSc) ? 4 : 8) : 0;
  static constexpr int kEpiWarps = kRegBalance ? 8 : 4;
  static constexpr int kEpiWarp0 = kRegBalance ? 4 : 2;
  static constexpr int kUnpackWarp0 = kEpiWarp0 + kEpiWarps;
  static constexpr int kThreads = (kUnpackWarp0 + kUnpackWarps) * 32;
  static constexpr int kRegsLight = (kWideSc || kTmemA || kWide) ? 24 : (kScale == SCALE_SC) ? 32 : 40;    // TMA / MMA warpgroup (subchannel: every register counts)
  static constexpr int kRegsUnpack = kWideSc ? 56 : (kTmemA || kWide) ? 72 : 80;
  static constexpr int kRegsEpilogue = kWideSc ? 168 : (kScale == SCALE_SC) ? 200 : 136;  // subchannel: 128 running sums + room to interleave
  // The most registers per thread the kernel can be launched with (what the compiler may use before the
  // re-balance).  setmaxnreg.dec must not name more than a warp currently has, setmaxnreg.inc not less: a
  // role whose target is at or above this cap raises its count, one below it lowers it, and the host checks
  // the compiled kernel's actual register count against both before the first launch.
  static constexpr int kCapRegs = (65536 / kThreads) / 8 * 8 > 255 ? 255 : (65536 / kThreads) / 8 * 8;
  static constexpr bool kUnpackRaises = kRegsUnpack >= kCapRegs;
  // registers the CTA needs after the re-balance; the host checks this against regs-per-thread x threads
  static constexpr int kRegPoolNeeded = kRegBalance ? (128 * kRegsLight + 256 * kRegsEpilogue + kUnpackWarps * 32 * kRegsUnpack) : 0;
  // A CTA of a pair holds one 128-wide block of B (the MMA reads the other one from the peer), so
  // its stages are a third smaller and more of them fit.
  static constexpr int kBBlocks = (k2Cta && !kWide) ? 1 : 2;
  static constexpr int kStages = kTmemA ? 7
                                 : kWide ? 2
                                 : kShortK ? 2
                                 : kInt4 ? (k2Cta ? 4 : 3)
                                         : (k2Cta ? 6 : 4);  // int8 UMMA stages
  static constexpr int kPkStages =
      kTmemA ? 4 : kWide ? 4 : kInt4 ? (k2Cta ? (kShortK ? 5 : 4) : 2) : 0; // packed staging stages (backward pairs: a group's reduction is
                                                                  // short, so what pays is TMA running five K blocks ahead across tiles:
                                                                  // 200.5 us with 3 + 3 stages, 190.1 with 2 + 4, 186.2 with 2 + 5)
  static constexpr int kA8Bytes = kTmemA ? 0 : BM * BK;     // 16 KB (none: A lives in TMEM)
  static constexpr int kB8Bytes = kBBlocks * NBLK * BK;     // 32 KB (pair: 16 KB)
  static constexpr int kStageBytes = kA8Bytes + kB8Bytes;
  static constexpr int kPkABytes = BM * BK / 2;             // 8 KB
  static constexpr int kPkBBytes = kBBlocks * NBLK * BK / 2;  // 16 KB (pair: 8 KB)
  static constexpr int kPkStageBytes = kPkABytes + kPkBBytes;
  static constexpr int kBarBytes = 512;
  // results leave through shared memory + TMA stores (per-channel kernels; 2 KB per epilogue warp)
  static constexpr bool kTmaStore = (kScale == SCALE_PC) ? (kOut != OUT_S32) : (kOut == OUT_BF16);
  static constexpr int kStagingSlots = kWide ? 1 : 2;
  // fp32 output of the backward kernels: two 4 KB slots per warp, so that a chunk is staged while TMA still
  // reads the previous one
  static constexpr int kF32Slots = kShortK ? 2 : 1;
  // per-channel: per warp 2 slots x 2 KB (bf16) or kF32Slots x 4 KB (fp32); subchannel: 2 KB per warp
  static constexpr int kStagingPerWarp =
      (kScale == SCALE_PC) ? (kOut == OUT_F32 ? kF32Slots * 4096 : kStagingSlots * 2048) : 2048;
  static constexpr int kStagingBytes = kTmaStore ? kEpiWarps * kStagingPerWarp : 0;
  // column scales as fp32: per-channel 256 per warp; subchannel 2 x 128 per warp (double-buffered by K-group)
  static constexpr int kScaleStripBytes = kEpiWarps * 1024;
  static constexpr int kSmemBytes =
      1024 + kStages * kStageBytes + kPkStages * kPkStageBytes + kStagingBytes + kScaleStripBytes + kBarBytes;
  static_assert(kSmemBytes <= 232448, "over the 227 KB of shared memory a CTA can have");
};

// FLAVOR_FUSED_SC (kFastSc, subchannel kernels only): the order of roundings of the per-K-group accumulation.
//   false: out += (f32(acc_g) * sa_g) * sb_g with every rounding of the reference (api.py:316-324): bit-identical;
//   true : out = fma(f32(acc_g) * sa_g, sb_g, out): the last multiply and the add share one rounding, and the
//          int -> float step costs nothing because the accumulators start from a bias in TMEM (see the epilogue).
//          Two instructions per element and K-group instead of four; results differ from the reference in the
//          last bits of the fp32 running sum, far inside the bf16 output tolerance.
template <bool kInt4, bool kAMn, bool kBMn, int kScale, int kEpi, int kOut, bool kMaskK, bool k2Cta = false, int kFlavor = FLAVOR_PLAIN>
__global__ void __launch_bounds__(KernelTraits<kInt4, kAMn, kBMn, kScale, kEpi, kOut, kMaskK, k2Cta, kFlavor>::kThreads, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using T = KernelTraits<kInt4, kAMn, kBMn, kScale, kEpi, kOut, kMaskK, k2Cta, kFlavor>;
  constexpr bool kFastSc = T::kFastSc;
  constexpr bool kTmemA = T::kTmemA;
  constexpr bool kTail = T::kTail;
  constexpr bool kWide = T::kWide;
  static_assert(!kFastSc || kScale == SCALE_SC, "the fused accumulation order belongs to the subchannel kernels");
  // accumulator buffer and barrier phase of the grp-th accumulator hand-over
  auto acc_buf = [](int grp) { return grp % T::kAccBufs; };
  auto acc_phase = [](int grp) -> uint32_t { return static_cast<uint32_t>((grp / T::kAccBufs) & 1); };
  constexpr int S = T::kStages;
  constexpr int PS = T::kPkStages;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  // layout: [S x (A8 | B8)] [PS x (pkA | pkB)] [output staging] [column-scale strips] [barriers]
  const uint32_t stage_base = smem_base;
  const uint32_t pk_base = stage_base + S * T::kStageBytes;
  const uint32_t bar_base = pk_base + PS * T::kPkStageBytes + T::kStagingBytes + T::kScaleStripBytes;
  uint8_t* bar_gen = smem_gen + S * T::kStageBytes + PS * T::kPkStageBytes + T::kStagingBytes + T::kScaleStripBytes;

  // barrier slots (8 bytes each)
  static_assert(S <= 8 && PS <= 8, "barrier slots are laid out for at most 8 stages");
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (8 + s); };
  auto pk_full_bar = [&](int s) { return bar_base + 8u * (16 + s); };
  auto pk_empty_bar = [&](int s) { return bar_base + 8u * (24 + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (32 + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (34 + b); };
  auto peer_full_bar = [&](int s) { return bar_base + 8u * (36 + s); };  // leader CTA of a pair only
  const uint32_t preload_bar = bar_base + 8u * 45;  // balanced tail: the owner segment's accumulator holds its neighbour's partial sum
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * 44);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * 44 + 4);
  // CTA pairs: the cluster is the scheduling unit; the leader (rank 0) issues the MMAs for both.
  const int cta_rank = k2Cta ? static_cast<int>(cluster_ctarank()) : 0;
  const int unit = k2Cta ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
  int tile0 = unit;
  int tile_step = k2Cta ? static_cast<int>(cluster_count_x()) : static_cast<int>(gridDim.x);
  // grouped forward with tasks built on the device: the task count is read here, not passed by the host
  int num_tiles = p.num_tasks_dev != nullptr ? min(*p.num_tasks_dev, p.tiles_m) * p.tiles_n : p.num_tiles;
  if (kTail && p.tail_units > 0) {
    // balanced tail: the roles walk this unit's segments
    tile0 = 0;
    tile_step = 1;
    num_tiles = p.tail_waves + (unit < p.tail_split * p.tail_rest ? 1 : 0);
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AbortCtx ctx{abort_flag, p.status};
  // a task list that did not fit its arrays leaves rows of the output unwritten: say so in the status word
  if (p.overflow_dev != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && *p.overflow_dev != 0 && p.status != nullptr &&
      p.status[0] == STATUS_OK) {
    p.status[1] = *p.num_tasks_dev;
    p.status[2] = 0;
    p.status[0] = STATUS_TASK_OVERFLOW;
  }
  // per-epilogue-warp 2 KB staging buffer of the TMA store path (warps 2..5 -> slots 0..3)
  const int epi_slot = (warp - T::kEpiWarp0) & (T::kEpiWarps - 1);
  uint8_t* stage_out = smem_gen + S * T::kStageBytes + PS * T::kPkStageBytes + epi_slot * T::kStagingPerWarp;
  float* sb_strip = reinterpret_cast<float*>(smem_gen + S * T::kStageBytes + PS * T::kPkStageBytes + T::kStagingBytes + epi_slot * 1024);
  const uint32_t stage_out_u32 = stage_base + S * T::kStageBytes + PS * T::kPkStageBytes + epi_slot * T::kStagingPerWarp;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), kInt4 ? T::kUnpackWarps : 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(peer_full_bar(s), 1);
    }
    for (int s = 0; s < PS; ++s) {
      mbar_init(pk_full_bar(s), 1);
      mbar_init(pk_empty_bar(s), T::kUnpackWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), (k2Cta ? 2 : 1) * T::kEpiWarps);  // pair: both CTAs' epilogue warps
    }
    mbar_init(preload_bar, (k2Cta ? 2 : 1) * T::kEpiWarps);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if constexpr (k2Cta) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (k2Cta) cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (T::kRegBalance) {
    if (warp < 4) reg_dealloc<T::kRegsLight>();  // all four warps of warpgroup 0, the idle ones included
  }

  // K-groups: number of K=32 MMA steps between accumulator hand-overs to the epilogue.
  // Per-channel: the whole tile is one group.
  const int mma_per_group = (kScale == SCALE_SC) ? (p.subchannel / 32) : 0x7FFFFFFF;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = tile0; t < num_tiles && ok; t += tile_step) {
        const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
        // wide tiles: this CTA's share of the tile's second 256 (or, for a 384-column tile, 128) columns
        const int wide_b1_x = w.n0 + BN + (w.tq ? NBLK / 2 : NBLK) * cta_rank;
        for (int kbl = 0; kbl < w.num_kb; ++kbl, ++it) {
          const int kb = kbl + w.kb0;  // K block of the whole reduction (a split-K slice starts past 0)
          if constexpr (kInt4) {
            const int s = it % PS;
            const uint32_t ph = (it / PS) & 1;
            if (!mbar_wait(pk_empty_bar(s), ph ^ 1u, ctx, 10)) { ok = false; break; }
            const uint32_t dst = pk_base + s * T::kPkStageBytes;
            mbar_arrive_expect_tx(pk_full_bar(s), T::kPkStageBytes);
            if constexpr (kAMn) {
              tma_load_2d(dst, &tmap_a, w.a_x, w.a_y + kb * (BK / 2), pk_full_bar(s));
            } else {
              tma_load_2d(dst, &tmap_a, w.a_x + kb * (BK / 2), w.a_y, pk_full_bar(s));
            }
            // a CTA of a pair brings one block of B: the leader the first, its peer the second
            const int nb0 = (k2Cta && cta_rank != 0) ? w.n1 : w.n0;
            if constexpr (kWide) {
              // this CTA's 128 columns of each of the tile's two 256-column halves
              tma_load_2d(dst + T::kPkABytes, &tmap_b, w.n0 + NBLK * cta_rank, w.b_y + kb * (BK / 2), pk_full_bar(s));
              tma_load_2d(dst + T::kPkABytes + T::kPkBBytes / 2, &tmap_b, wide_b1_x, w.b_y + kb * (BK / 2), pk_full_bar(s));
            } else if constexpr (kBMn) {
              tma_load_2d(dst + T::kPkABytes, &tmap_b, nb0, w.b_y + kb * (BK / 2), pk_full_bar(s));
              if constexpr (!k2Cta)
                tma_load_2d(dst + T::kPkABytes + T::kPkBBytes / 2, &tmap_b, w.n1,
                            w.b_y + kb * (BK / 2), pk_full_bar(s));
            } else {
              tma_load_2d(dst + T::kPkABytes, &tmap_b, kb * (BK / 2), w.b_y + nb0, pk_full_bar(s));
              if constexpr (!k2Cta)
                tma_load_2d(dst + T::kPkABytes + T::kPkBBytes / 2, &tmap_b, kb * (BK / 2), w.b_y + w.n1,
                            pk_full_bar(s));
            }
          } else {
            const int s = it % S;
            const uint32_t ph = (it / S) & 1;
            if (!mbar_wait(empty_bar(s), ph ^ 1u, ctx, 11)) { ok = false; break; }
            const uint32_t dst = stage_base + s * T::kStageBytes;
            mbar_arrive_expect_tx(full_bar(s), T::kStageBytes);
            if constexpr (kAMn) {
              tma_load_2d(dst, &tmap_a, w.a_x, w.a_y + kb * BK, full_bar(s));
            } else {
              tma_load_2d(dst, &tmap_a, w.a_x + kb * BK, w.a_y, full_bar(s));
            }
            const int nb0 = (k2Cta && cta_rank != 0) ? w.n1 : w.n0;
            if constexpr (kBMn) {
              tma_load_2d(dst + T::kA8Bytes, &tmap_b, nb0, w.b_y + kb * BK, full_bar(s));
              if constexpr (!k2Cta)
                tma_load_2d(dst + T::kA8Bytes + T::kB8Bytes / 2, &tmap_b, w.n1, w.b_y + kb * BK,
                            full_bar(s));
            } else {
              tma_load_2d(dst + T::kA8Bytes, &tmap_b, kb * BK, w.b_y + nb0, full_bar(s));
              if constexpr (!k2Cta)
                tma_load_2d(dst + T::kA8Bytes + T::kB8Bytes / 2, &tmap_b, kb * BK, w.b_y + w.n1,
                            full_bar(s));
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the schedule and waits on barriers together (so that loop control
    // stays warp-uniform); one elected lane issues the MMAs and the commits.
    constexpr uint32_t idesc = umma_idesc_i8(k2Cta ? 2 * BM : BM, BN, kAMn, kBMn);
    // single CTA or pair: the MMA, the commit, and the wait for operands (a pair's leader also waits
    // for the peer's "stage full" signal, forwarded by the peer's warp 1)
    auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t acc_flag) {
      if constexpr (k2Cta) umma_i8_pair(d, da, db, idesc, acc_flag);
      else umma_i8(d, da, db, idesc, acc_flag);
    };
    auto commit = [&](uint32_t bar) {
      if constexpr (k2Cta) umma_commit_pair(bar);
      else umma_commit(bar);
    };
    auto wait_operands = [&](int s, uint32_t ph) -> bool {
      bool got = mbar_wait(full_bar(s), ph, ctx, 20);
      if constexpr (k2Cta) got = got && mbar_wait(peer_full_bar(s), ph, ctx, 22);
      return got;
    };
    auto wait_acc_empty = [&](int b, uint32_t ph) -> bool { return mbar_wait(acc_empty_bar(b), ph, ctx, 21); };
    if (k2Cta && cta_rank != 0) {
      // Peer CTA of a pair: no MMAs are issued here.  Forward "my stage s is full" to the leader.
      int it = 0;
      bool ok = true;
      for (int t = tile0; t < num_tiles && ok; t += tile_step) {
        const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
        for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(full_bar(s), ph, ctx, 23))) { ok = false; break; }
          if (elect_one()) {
            mbar_arrive_cluster(map_to_cta(peer_full_bar(s), 0));
          }
          __syncwarp();
        }
      }
    } else {
    // descriptor = {lo: start address >> 4 | LBO >> 4 << 16, hi: SBO >> 4 | version | swizzle}
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
    constexpr uint32_t kALboField = (kAMn ? (BK * NBLK) >> 4 : 1u) << 16;
    constexpr uint32_t kBLboField = (kBMn ? (BK * NBLK) >> 4 : 1u) << 16;
    constexpr uint32_t kAStep = (kAMn ? 32 * NBLK : 32) >> 4;   // one K=32 step, in 16-byte units
    constexpr uint32_t kBStep = (kBMn ? 32 * NBLK : 32) >> 4;
    const uint32_t a_lo0 = ((stage_base & 0x3FFFFu) >> 4) | kALboField;
    const uint32_t b_lo0 = (((stage_base + T::kA8Bytes) & 0x3FFFFu) >> 4) | kBLboField;
    auto make_desc = [&](uint32_t lo) -> uint64_t { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
    int it = 0;
    int grp = 0;  // accumulator hand-over counter (one per K-group)
    bool ok = true;
    for (int t = tile0; t < num_tiles && ok; t += tile_step) {
      const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
      const int total_mma = (w.k_len + 31) / 32;  // K=32 steps that hold real data
      // 384-column tiles: the second MMA covers 128 columns, the first 64 of each CTA's second block of B
      const uint32_t idesc_second = (kWide && w.tq) ? umma_idesc_i8(k2Cta ? 2 * BM : BM, NBLK, kAMn, kBMn) : idesc;
      if constexpr (kScale == SCALE_PC) {
        if (w.num_kb == 0) continue;
        const int b = acc_buf(grp);
        if (!__all_sync(0xFFFFFFFFu, wait_acc_empty(b, acc_phase(grp) ^ 1u))) { ok = false; break; }
        // balanced tail: the epilogue warps have put the neighbour's partial sum into this buffer (a unit owns at
        // most one such tile, so the barrier is used once); the MMAs add onto it
        const uint32_t onto = (kTail && w.part == PART_OWNER && p.tail_waves > 0) ? 1u : 0u;
        if (onto != 0u) {
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(preload_bar, 0u, ctx, 24))) { ok = false; break; }
          tc_fence_after_sync();
        }
        for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!__all_sync(0xFFFFFFFFu, wait_operands(s, ph))) { ok = false; break; }
          tc_fence_after_sync();
          if (elect_one()) {
            const uint32_t a_lo = a_lo0 + s * (T::kStageBytes >> 4);
            const uint32_t b_lo = b_lo0 + s * (T::kStageBytes >> 4);
            const int left = total_mma - kb * (BK / 32);
#pragma unroll
            for (int k = 0; k < BK / 32; ++k) {
              if (k < left) {
                if constexpr (kTmemA)
                  umma_i8_pair_tmem_a(tmem_base + b * BN, tmem_base + T::kTmemAStage0 + s * 32 + k * 8,
                                      make_desc(b_lo + k * kBStep), idesc, ((kb | k) != 0 ? 1u : 0u) | onto);
                else
                  mma(tmem_base + b * BN, make_desc(a_lo + k * kAStep), make_desc(b_lo + k * kBStep),
                      ((kb | k) != 0 ? 1u : 0u) | onto);
                if constexpr (kWide)  // the tile's second 256 columns: the same A, this pair's second blocks of B
                  umma_i8_pair(tmem_base + BN, make_desc(a_lo + k * kAStep), make_desc(b_lo + ((T::kB8Bytes / 2) >> 4) + k * kBStep),
                               idesc_second, ((kb | k) != 0 ? 1u : 0u));
              }
            }
            commit(empty_bar(s));
#ifndef B200_TEST_DROP_ACC_FULL_SIGNAL
            if (kb == w.num_kb - 1) commit(acc_full_bar(b));
#endif
          }
          __syncwarp();
        }
        ++grp;
      } else if (mma_per_group >= BK / 32) {
        // K-groups of 128 or 256: a K block never straddles two groups, so a block is issued in
        // one go exactly like the per-channel case, with the accumulator hand-over at group ends
        const int kb_per_group = mma_per_group / (BK / 32);
        for (int kb = 0; kb < w.num_kb && ok; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          const int b = grp & 1;
          const bool group_start = (kb % kb_per_group) == 0;
          const bool group_end = ((kb + 1) % kb_per_group) == 0 || kb == w.num_kb - 1;
          if (group_start) {
            // fused order: the epilogue warps arm both buffers before the first group, which is phase 0 of the
            // "empty" barriers; otherwise the buffers start out free
            const uint32_t free_parity = kFastSc ? ((grp >> 1) & 1) : (((grp >> 1) & 1) ^ 1u);
            if (!__all_sync(0xFFFFFFFFu, wait_acc_empty(b, free_parity))) { ok = false; break; }
          }
          if (!__all_sync(0xFFFFFFFFu, wait_operands(s, ph))) { ok = false; break; }
          tc_fence_after_sync();
          if (elect_one()) {
            const uint32_t a_lo = a_lo0 + s * (T::kStageBytes >> 4);
            const uint32_t b_lo = b_lo0 + s * (T::kStageBytes >> 4);
            const int left = total_mma - kb * (BK / 32);
#pragma unroll
            for (int k = 0; k < BK / 32; ++k) {
              if (k < left)
                mma(tmem_base + b * BN, make_desc(a_lo + k * kAStep), make_desc(b_lo + k * kBStep),
                    (!kFastSc && group_start && k == 0) ? 0u : 1u);  // fused order: always onto the bias
            }
            commit(empty_bar(s));
            if (group_end) commit(acc_full_bar(b));
          }
          __syncwarp();
          if (group_end) ++grp;
        }
      } else if constexpr (!k2Cta) {
        // K-groups of 32 or 64 (single-CTA kernels only; the host never pairs CTAs for them)
        int j = 0;  // MMA step within the tile
        for (int kb = 0; kb < w.num_kb && ok; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(full_bar(s), ph, ctx, 20))) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (T::kStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + s * (T::kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k, ++j) {
            if (j >= total_mma) break;
            const int in_group = j % mma_per_group;
            const int b = grp & 1;
            if (in_group == 0) {
              const uint32_t free_parity = kFastSc ? ((grp >> 1) & 1) : (((grp >> 1) & 1) ^ 1u);
              if (!__all_sync(0xFFFFFFFFu, mbar_wait(acc_empty_bar(b), free_parity, ctx, 21))) { ok = false; break; }
              tc_fence_after_sync();
            }
            const bool group_end = (in_group == mma_per_group - 1) || (j == total_mma - 1);
            if (elect_one()) {
              umma_i8(tmem_base + b * BN, make_desc(a_lo + k * kAStep), make_desc(b_lo + k * kBStep), idesc,
                      (kFastSc || in_group != 0) ? 1u : 0u);
              if (group_end) umma_commit(acc_full_bar(b));
            }
            __syncwarp();
            if (group_end) ++grp;
          }
          if (ok) {
            if (elect_one()) umma_commit(empty_bar(s));
            __syncwarp();
          }
        }
      }
    }
    }  // leader / single CTA
  } else if (warp >= T::kEpiWarp0 && warp < T::kUnpackWarp0) {
    // ------------------------------------------------------------------ epilogue
    if constexpr (T::kRegBalance) reg_alloc<T::kRegsEpilogue>();
    const int e = warp - T::kEpiWarp0;
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int half = e >> 2;                 // column half (subchannel mode runs 8 warps)
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    int grp = 0;
    // hand accumulator buffer b back to the MMA issuer (of a pair: the leader CTA's)
    auto release_acc = [&](int b) {
      if constexpr (k2Cta) mbar_arrive_cluster(map_to_cta(acc_empty_bar(b), 0));
      else mbar_arrive(acc_empty_bar(b));
    };
    int store_count = 0;  // TMA stores issued by this warp (selects the staging slot)
    bool ok = true;
    // Balanced tail: the segment this unit owns together with its right-hand neighbour (always its last one), and the
    // segment after whose read-out this warp writes the neighbour's partial sum into the accumulator buffer that the
    // owner segment will use (the buffer's previous user; < 0: nobody used it before, preload before the first tile).
    int owner_seg = -1;
    if constexpr (kTail) {
      if (p.tail_units > 0 && p.tail_waves > 0 && unit < p.tail_rest) owner_seg = num_tiles - 1;
    }
    const int preload_after = owner_seg - T::kAccBufs;
    // Slot layout: 16-byte piece i of chunk c of row r at int4 index ((c * 8 + i) * 128 + r): a warp's 32 rows read or
    // write 512 contiguous bytes per instruction.  Producer and owner are the same kernel, so they agree on it.
    // Waits until every other part of this unit's rest tile has been written; false when the wait was abandoned.
    // The flags return to zero inside the launch, so that the next launch on the same workspace needs no memset
    // between kernels: every warp that has seen a flag complete counts itself in the word beside it, and the last of
    // the unit's epilogue warps to do so clears both.
    auto partners_ready = [&]() -> bool {
      bool got = true;
      if (lane == 0) {
        for (int part = 1; part < p.tail_split && got; ++part) {
          int* flag = p.tail_flags + ((part * p.tail_rest + unit) * 2 + cta_rank) * 2;
          got = flag_wait(flag, T::kEpiWarps, ctx, 32);
          if (got && atomicAdd(flag + 1, 1) == T::kEpiWarps - 1) {
            flag[1] = 0;
            __threadfence();
            flag[0] = 0;
          }
        }
      }
      return __all_sync(0xFFFFFFFFu, got);
    };
    // this thread's row of the first other part's slot, and the distance (in int4) from one part's slot to the next
    const int4* first_part = reinterpret_cast<const int4*>(p.tail_partials) +
                             static_cast<long long>((p.tail_rest + unit) * 2 + cta_rank) * (BM * BN / 4) + row_in_tile;
    const long long part_stride = static_cast<long long>(p.tail_rest) * 2 * (BM * BN / 4);
    constexpr int kRawChunks = 8 / (T::kEpiWarps / 4);
    // With a full wave before it, the owner part starts from the other parts' sum: this warp writes its share of the
    // sum into the accumulator buffer the owner part will use, right after it has read that buffer's previous tile.
    auto preload_partner = [&]() -> bool {
      const int b = acc_buf(owner_seg);
      if (!partners_ready()) return false;
      tail_sum_into_tmem(tmem_base + lane_addr + b * BN, first_part, part_stride, p.tail_split - 1, half * kRawChunks,
                         (half + 1) * kRawChunks, false);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (k2Cta) mbar_arrive_cluster(map_to_cta(preload_bar, 0));
        else mbar_arrive(preload_bar);
      }
      return true;
    };
    if constexpr (kTail) {
      if (owner_seg >= 0 && preload_after < 0) ok = preload_partner();
    }
    // Fused order.  For |x| <= 2^22 the float with bit pattern 0x4B400000 + x is exactly 1.5 * 2^23 + x.  The
    // accumulators therefore start from the integer 0x4B400000 instead of 0 (the tensor core adds the products onto
    // whatever TMEM holds): what comes back from TMEM is already the float 1.5 * 2^23 + acc, no conversion, no
    // integer add.  The epilogue warps write the bias: once into both buffers here, and again over every chunk
    // they have read, before they hand the buffer back.
    constexpr uint32_t kBiasBits = 0x4B400000u;
    // first TMEM column of this warp's c-th 16-column chunk (the order of its running sums)
    auto sc_chunk_col = [&](int c) -> int {
      if constexpr (kEpi == EPI_SWIGLU) return (c < 4) ? (64 * half + 16 * c) : (NBLK + 64 * half + 16 * (c - 4));
      else return 128 * half + 16 * c;
    };
    if constexpr (kFastSc) {
#pragma unroll
      for (int b = 0; b < 2; ++b) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_st_fill_32x32b_x16(tmem_base + lane_addr + b * BN + sc_chunk_col(c), kBiasBits);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        release_acc(0);
        release_acc(1);
      }
    }
    // Columns of the 256-wide accumulator this warp owns:
    //   per-channel, 4 warps: all 256 (SwiGLU: up 0..127 with gate 128..255)
    //   subchannel, 8 warps : plain -> [128*half, +128); SwiGLU -> up [64*half,+64) with gate 128+[64*half,+64)
    constexpr int kOwnCols = (kScale == SCALE_SC) ? 128 : 256;
    for (int t = tile0; t < num_tiles && ok; t += tile_step) {
      const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
      const int row = w.out_row0 + row_in_tile;
      const bool row_ok = (row >= w.row_lo) && (row < w.row_hi);
      const long long sa_row = w.sa_off + static_cast<long long>(row) * (kScale == SCALE_SC ? p.scale_cols : 1);

      if constexpr (kScale == SCALE_PC) {
        float sa_pre = 0.f;  // the row's scale; for int4 divided by the 256 the accumulator carries (exact)
        if constexpr (kOut != OUT_S32) {
          if (row_ok) sa_pre = __bfloat162float(p.a_scale[sa_row]) * (kInt4 ? (1.0f / 256.0f) : 1.0f);
        }
        const bool zero_tile = (w.num_kb == 0);  // nothing to reduce (empty group): the result is zero
        // Column scales of the tile, once per tile, into this warp's strip of shared memory as fp32
        // (lane l brings the 8 columns 8l..8l+7 of the 256-wide accumulator).  One global-load
        // latency per tile, overlapped with the wait for the accumulator.
        if constexpr (kOut != OUT_S32) {
          const int tc = 8 * lane;
          // wide tiles: the strip holds the scales of this warp's own 256 columns of the 512
          const int bcol = kWide ? (w.n0 + BN * half + tc) : (tc < NBLK) ? (w.n0 + tc) : (w.n1 + tc - NBLK);  // column of b_scale
          const int ocol = kWide ? bcol : (tc < NBLK || kEpi != EPI_SWIGLU) ? (w.n0 + tc) : (w.n0 + tc - NBLK);  // output column
          const long long idx = w.sb_off + bcol;
          float f[8];
          if (ocol + 8 <= p.N && (idx & 7) == 0) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(p.b_scale + idx));
            const uint32_t ws[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) {
              f[2 * k2] = __uint_as_float(ws[k2] << 16);
              f[2 * k2 + 1] = __uint_as_float(ws[k2] & 0xFFFF0000u);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = (ocol + i < p.N) ? __bfloat162float(p.b_scale[idx + i]) : 0.f;
          }
          __syncwarp();  // every lane is done reading the previous tile's scales
          reinterpret_cast<float4*>(sb_strip)[2 * lane] = make_float4(f[0], f[1], f[2], f[3]);
          reinterpret_cast<float4*>(sb_strip)[2 * lane + 1] = make_float4(f[4], f[5], f[6], f[7]);
          __syncwarp();
        }
        int b = 0;
        if (!zero_tile) {
          b = acc_buf(grp);
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(acc_full_bar(b), acc_phase(grp), ctx, 30))) { ok = false; break; }
          tc_fence_after_sync();
        }
        // Balanced tail.  A producer segment ends here: its raw accumulators (the exact s32 sums of the tile's last
        // K blocks) go to the partial-sum slot, 128 bytes per thread and chunk, and each warp announces its share.
        // Balanced tail.  A producer segment ends here: its raw accumulators (the exact s32 sums of the tile's last
        // K blocks) go to this unit's partial-sum slot and each warp announces its share.
        if (kTail && w.part == PART_PRODUCER) {
          int4* dst = reinterpret_cast<int4*>(p.tail_partials) + static_cast<long long>(w.part_slot * 2 + cta_rank) * (BM * BN / 4) + row_in_tile;
          uint32_t r[32];
#pragma unroll 1
          for (int c = half * kRawChunks; c < (half + 1) * kRawChunks; ++c) {
            tmem_ld_32x32b_x32(tmem_base + lane_addr + b * BN + 32 * c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i)
              __stcg(dst + (c * 8 + i) * BM, make_int4(static_cast<int>(r[4 * i]), static_cast<int>(r[4 * i + 1]),
                                                       static_cast<int>(r[4 * i + 2]), static_cast<int>(r[4 * i + 3])));
          }
          if (kTail && t == preload_after && !preload_partner()) { ok = false; break; }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) release_acc(b);
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(p.tail_flags + (w.part_slot * 2 + cta_rank) * 2, 1);
          ++grp;
          continue;
        }
        // TMA store path: the warp's 32 rows must all be rows this tile owns (rows past the end of a
        // dense output are clipped by the tensor map itself)
        const int wrow0 = w.out_row0 + q * 32;
        const bool use_tma = T::kTmaStore && p.tma_store != 0 &&
                             ((p.mode == MODE_DENSE && p.k_slices == 1) || (wrow0 >= w.row_lo && wrow0 + 32 <= w.row_hi));
        const uint32_t acc_addr = tmem_base + lane_addr + b * BN;

        // one 32-column chunk: scale, activation, store
        // no full wave before the owner part (fewer tiles than units): the other parts run at the same time, so their
        // sums are added here, after the MMAs, instead of being preloaded
        if (kTail && w.part == PART_OWNER && p.tail_waves == 0) {
          if (!partners_ready()) { ok = false; break; }
          tail_sum_into_tmem(tmem_base + lane_addr + b * BN, first_part, part_stride, p.tail_split - 1, half * kRawChunks,
                             (half + 1) * kRawChunks, true);
        }
        auto process = [&](uint32_t (&r)[32], int c) {
          const int col0 = w.n0 + 32 * c;  // output column of this chunk

          if constexpr (kOut == OUT_S32) {
            if (row_ok) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = col0 + i;
                if (col < p.N) {
                  int a = static_cast<int>(r[i]);
                  if constexpr (kInt4) a >>= 8;
                  reinterpret_cast<int*>(p.out)[w.out_off + static_cast<long long>(row) * p.ldc + col] = a;
                }
              }
            }
          } else {
            // (f32(acc) * sa) * sb, two roundings, two elements per instruction.  An int4 accumulator holds 256 * sum:
            // converting it as it is and multiplying by sa / 256 (`sa_pre`) gives the bits of f32(sum) * sa, because a
            // power of two scales the convert's rounding and the product's exactly.
            float v[32];
            const float2 sa2 = make_float2(sa_pre, sa_pre);
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 sb4 = reinterpret_cast<const float4*>(sb_strip)[8 * (kWide ? (c & 7) : c) + i4];  // broadcast read
              const float2 lo = __fmul2_rn(__fmul2_rn(make_float2(static_cast<float>(static_cast<int>(r[4 * i4])),
                                                                  static_cast<float>(static_cast<int>(r[4 * i4 + 1]))), sa2),
                                           make_float2(sb4.x, sb4.y));
              const float2 hi = __fmul2_rn(__fmul2_rn(make_float2(static_cast<float>(static_cast<int>(r[4 * i4 + 2])),
                                                                  static_cast<float>(static_cast<int>(r[4 * i4 + 3]))), sa2),
                                           make_float2(sb4.z, sb4.w));
              v[4 * i4] = lo.x;
              v[4 * i4 + 1] = lo.y;
              v[4 * i4 + 2] = hi.x;
              v[4 * i4 + 3] = hi.y;
            }
            if constexpr (kEpi == EPI_SWIGLU) {
              uint32_t g[32];
              tmem_ld_32x32b_x32(acc_addr + NBLK + 32 * c, g);
              tmem_ld_wait();

#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float gate = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(g[i])), sa_pre), sb_strip[NBLK + 32 * c + i]);
                v[i] = v[i] * (gate / (1.0f + __expf(-gate)));
              }
            } else if constexpr (kEpi == EPI_RELU2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float x = fmaxf(v[i], 0.f);
                v[i] = x * x;
              }
            }
            if (use_tma) {
              // stage 32 rows in shared memory, then one TMA store writes whole lines; columns past N
              // are clipped by the tensor map.  bf16: 64 B per row, two 2 KB slots, 64-byte swizzle
              // (chunk ^ ((row >> 1) & 3)).  fp32: 128 B per row, one 4 KB slot, 128-byte swizzle.
              if constexpr (kOut == OUT_BF16) {
                const int slot = T::kStagingSlots == 2 ? (store_count & 1) : 0;
                ++store_count;
                uint8_t* dst = stage_out + slot * 2048 + lane * 64;
                const int sw = (lane >> 1) & 3;
                if (lane == 0) {
                  if constexpr (T::kStagingSlots == 2) bulk_wait_read_keep1();
                  else bulk_wait_read_all();
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 pk;
                  __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
                  __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                  __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                  pk.x = *reinterpret_cast<uint32_t*>(&h0);
                  pk.y = *reinterpret_cast<uint32_t*>(&h1);
                  pk.z = *reinterpret_cast<uint32_t*>(&h2);
                  pk.w = *reinterpret_cast<uint32_t*>(&h3);
                  *reinterpret_cast<uint4*>(dst + ((i ^ sw) << 4)) = pk;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&tmap_c, stage_out_u32 + slot * 2048, col0 * 2, w.out_row_base + wrow0);
                  bulk_commit_group();
                }
              } else if constexpr (T::kF32Slots == 2) {
                const int slot = store_count & 1;
                ++store_count;
                uint8_t* dst = stage_out + slot * 4096 + lane * 128;
                const int sw = lane & 7;
                if (lane == 0) bulk_wait_read_keep<1>();
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  uint4 pk;
                  pk.x = __float_as_uint(v[4 * i + 0]);
                  pk.y = __float_as_uint(v[4 * i + 1]);
                  pk.z = __float_as_uint(v[4 * i + 2]);
                  pk.w = __float_as_uint(v[4 * i + 3]);
                  *reinterpret_cast<uint4*>(dst + ((i ^ sw) << 4)) = pk;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&tmap_c, stage_out_u32 + slot * 4096, col0 * 4, w.out_row_base + wrow0);
                  bulk_commit_group();
                }
              } else {
                uint8_t* dst = stage_out + lane * 128;
                const int sw = lane & 7;
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  uint4 pk;
                  pk.x = __float_as_uint(v[4 * i + 0]);
                  pk.y = __float_as_uint(v[4 * i + 1]);
                  pk.z = __float_as_uint(v[4 * i + 2]);
                  pk.w = __float_as_uint(v[4 * i + 3]);
                  *reinterpret_cast<uint4*>(dst + ((i ^ sw) << 4)) = pk;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  tma_store_2d(&tmap_c, stage_out_u32, col0 * 4, w.out_row_base + wrow0);
                  bulk_commit_group();
                }
              }
            } else if (row_ok) {
              const long long o = w.out_off + static_cast<long long>(row) * p.ldc + col0;
              if constexpr (kOut == OUT_BF16) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
                if (col0 + 32 <= p.N && (p.ldc % 8 == 0)) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2);
                    pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    reinterpret_cast<uint4*>(dst)[i] = pk;
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) dst[i] = __float2bfloat16_rn(v[i]);
                }
              } else {
                float* dst = reinterpret_cast<float*>(p.out) + o;
                if (col0 + 32 <= p.N && (p.ldc % 4 == 0)) {
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) dst[i] = v[i];
                }
              }
            }
          }
        };

        constexpr int kAllChunks = (kEpi == EPI_SWIGLU) ? 4 : kWide ? 16 : 8;
        // with eight epilogue warps, the two warps of a lane quarter split the chunks between them
        constexpr int kOutChunks = kAllChunks / (T::kEpiWarps / 4);
        const int c_first = half * kOutChunks;
        const int c_end = c_first + ((kWide && w.tq && half == 1) ? kOutChunks / 2 : kOutChunks);  // 384 columns: chunks 8 .. 11
        // two register sets: the TMEM read of the next chunk is in flight while this one is processed
        uint32_t ra[32], rb[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) { ra[i] = 0u; rb[i] = 0u; }
        if (!zero_tile && kOutChunks > 0) tmem_ld_32x32b_x32(acc_addr + 32 * c_first, ra);
#pragma unroll 1
        for (int c = c_first; c < c_end; c += 2) {
          if (!zero_tile) {
            tmem_ld_wait();
            tmem_ld_fence(ra);
            tmem_ld_32x32b_x32(acc_addr + 32 * (c + 1), rb);
          }
          process(ra, c);
          if (!zero_tile) {
            tmem_ld_wait();
            tmem_ld_fence(rb);
            if (c + 2 < c_end) {
              tmem_ld_32x32b_x32(acc_addr + 32 * (c + 2), ra);
            } else if constexpr (kEpi != EPI_SWIGLU) {
              // the warp's last chunk is in registers: hand the accumulator back before processing it (the SwiGLU
              // epilogue still reads its gate columns while it processes)
              if (kTail && t == preload_after && !preload_partner()) ok = false;
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) release_acc(b);
            }
          }
          process(rb, c + 1);
        }
        if (!zero_tile) {
          if constexpr (kEpi == EPI_SWIGLU) {
            if (kTail && t == preload_after && !preload_partner()) ok = false;
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release_acc(b);
          }
          ++grp;
        }
      } else {
        // ---------------------------------------------------------------- subchannel scales
        // Running fp32 sums of the warp's 128 accumulator columns stay in registers:
        //   out += (f32(acc_g) * sa_g) * sb_g   for K-groups g in ascending order, out starting at 0.
        // int -> float without a convert instruction: for |x| <= 2^22 the float with bit pattern
        // 0x4B400000 + x is exactly 1.5 * 2^23 + x, so fma(that, sa, -(1.5 * 2^23) * sa) is the single
        // rounding of x * sa (the subtrahend is exact: sa has 8 significant bits).  A K-group has at
        // most 256 terms, |x| <= 256 * 64 * 256 = 2^22 (int4, values carried as 16 v) or 127^2 * 256.
        // For int4 the accumulator holds 256 * sum; sa is pre-multiplied by 2^-8, which is exact.
        constexpr uint32_t kMagicBits = 0x4B400000u;
        constexpr float kMagic = 12582912.0f;
        constexpr float kPreScale = kInt4 ? (1.0f / 256.0f) : 1.0f;
        float acc[kOwnCols];
#pragma unroll
        for (int i = 0; i < kOwnCols; ++i) acc[i] = 0.f;
        const int total_mma = (w.k_len + 31) / 32;
        const int num_groups = (total_mma + mma_per_group - 1) / mma_per_group;

        // Column scales: strip entry j (0..127) belongs to accumulator column j of this warp.
        // Lane l owns entries 4l..4l+3 (always on one side of the up / gate split).
        const int j0 = 4 * lane;
        int bcol, ocol;  // column of b_scale, output column (for the N edge)
        if constexpr (kEpi == EPI_SWIGLU) {
          const int tc = 64 * half + (j0 & 63);
          bcol = (j0 < 64) ? (w.n0 + tc) : (w.n1 + tc);
          ocol = w.n0 + tc;
        } else {
          const int tc = 128 * half + j0;
          bcol = (tc < NBLK) ? (w.n0 + tc) : (w.n1 + tc - NBLK);
          ocol = w.n0 + tc;
        }
        auto load_sb = [&](int gi, float (&f)[4]) {
          const long long idx = w.sb_off + static_cast<long long>(gi) * p.lds_b + bcol;
          if (ocol + 4 <= p.N && (idx & 3) == 0) {
            const uint2 x = __ldg(reinterpret_cast<const uint2*>(p.b_scale + idx));
            f[0] = __uint_as_float(x.x << 16);
            f[1] = __uint_as_float(x.x & 0xFFFF0000u);
            f[2] = __uint_as_float(x.y << 16);
            f[3] = __uint_as_float(x.y & 0xFFFF0000u);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = (ocol + i < p.N) ? __bfloat162float(p.b_scale[idx + i]) : 0.f;
          }
        };
        auto load_sa = [&](int gi) -> float {
          return row_ok ? __bfloat162float(p.a_scale[sa_row + gi]) * kPreScale : 0.f;
        };
        float sb_next[4] = {0.f, 0.f, 0.f, 0.f};
        float sa_next = 0.f;
        if (num_groups > 0) {
          load_sb(0, sb_next);
          sa_next = load_sa(0);
        }
        for (int gi = 0; gi < num_groups && ok; ++gi, ++grp) {
          // publish this group's column scales (fetched one group ago), then fetch the next group's
          float* strip = sb_strip + (gi & 1) * 128;
          __syncwarp();
          *reinterpret_cast<float4*>(strip + j0) = make_float4(sb_next[0], sb_next[1], sb_next[2], sb_next[3]);
          const float sa = sa_next;
          if (gi + 1 < num_groups) {
            load_sb(gi + 1, sb_next);
            sa_next = load_sa(gi + 1);
          }
          __syncwarp();
          const int b = grp & 1;
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(acc_full_bar(b), (grp >> 1) & 1, ctx, 31))) { ok = false; break; }
          tc_fence_after_sync();
          const float csa = -(kMagic * sa);
          if constexpr (kFastSc) {
            // two register sets: the TMEM read of the next chunk is in flight while this one is accumulated
            const uint32_t buf = tmem_base + lane_addr + b * BN;
            uint32_t ra[16], rb[16];
            tmem_ld_32x32b_x16(buf + sc_chunk_col(0), ra);
            // packed fp32 (two elements per instruction): the stream is bound by issue slots, which it shares
            // with the unpack warps, not by the fp32 pipe
            const float2 sa2 = make_float2(sa, sa), csa2 = make_float2(csa, csa);
            auto accumulate = [&](const uint32_t (&r)[16], int c) {
#pragma unroll
              for (int i4 = 0; i4 < 4; ++i4) {
                const float4 s4 = *reinterpret_cast<const float4*>(strip + 16 * c + 4 * i4);  // broadcast read
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                  const int j = 16 * c + 4 * i4 + 2 * h2;
                  const float2 y = make_float2(__uint_as_float(r[4 * i4 + 2 * h2]), __uint_as_float(r[4 * i4 + 2 * h2 + 1]));
                  const float2 sv = h2 == 0 ? make_float2(s4.x, s4.y) : make_float2(s4.z, s4.w);
                  const float2 t2 = __ffma2_rn(y, sa2, csa2);                              // = acc * sa, one rounding
                  const float2 sum = __ffma2_rn(t2, sv, make_float2(acc[j], acc[j + 1]));
                  acc[j] = sum.x;
                  acc[j + 1] = sum.y;
                }
              }
            };
#pragma unroll
            for (int c = 0; c < kOwnCols / 16; c += 2) {
              tmem_ld_wait();
              tmem_ld_fence16(ra);
              tmem_st_fill_32x32b_x16(buf + sc_chunk_col(c), kBiasBits);      // chunk c is in registers: re-arm it
              tmem_ld_32x32b_x16(buf + sc_chunk_col(c + 1), rb);
              accumulate(ra, c);
              tmem_ld_wait();
              tmem_ld_fence16(rb);
              tmem_st_fill_32x32b_x16(buf + sc_chunk_col(c + 1), kBiasBits);
              if (c + 2 < kOwnCols / 16) {
                tmem_ld_32x32b_x16(buf + sc_chunk_col(c + 2), ra);
              } else {
                // everything is read and re-armed: hand the buffer back before the last chunk's arithmetic
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) release_acc(b);
              }
              accumulate(rb, c + 1);
            }
          } else {
#pragma unroll
          for (int c = 0; c < kOwnCols / 16; ++c) {
            // 16 columns at a time; accumulator columns of this warp in strip order
            const int tcol = sc_chunk_col(c);
            uint32_t r[16];
            tmem_ld_32x32b_x16(tmem_base + lane_addr + b * BN + tcol, r);
            tmem_ld_wait();
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
              const float4 s4 = *reinterpret_cast<const float4*>(strip + 16 * c + 4 * i4);  // broadcast read
              const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int k2 = 0; k2 < 4; ++k2) {
                const float y = __uint_as_float(r[4 * i4 + k2] + kMagicBits);
                const float t2 = __fmaf_rn(y, sa, csa);
                acc[16 * c + 4 * i4 + k2] = __fadd_rn(acc[16 * c + 4 * i4 + k2], __fmul_rn(t2, sv[k2]));
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) release_acc(b);
          }
        }
        if (!ok) break;
        // activation + store, 32 output columns at a time
        const int wrow0 = w.out_row0 + q * 32;
        const bool use_tma = T::kTmaStore && p.tma_store != 0 &&
                             ((p.mode == MODE_DENSE && p.k_slices == 1) || (wrow0 >= w.row_lo && wrow0 + 32 <= w.row_hi));
        constexpr int kOutChunksSc = (kEpi == EPI_SWIGLU) ? 2 : 4;
#pragma unroll
        for (int c = 0; c < kOutChunksSc; ++c) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = acc[32 * c + i];
            if constexpr (kEpi == EPI_SWIGLU) {
              const float gate = acc[64 + 32 * c + i];
              x = x * (gate / (1.0f + __expf(-gate)));
            } else if constexpr (kEpi == EPI_RELU2) {
              x = fmaxf(x, 0.f);
              x = x * x;
            }
            v[i] = x;
          }
          const int ocol0 = w.n0 + ((kEpi == EPI_SWIGLU) ? 64 * half : 128 * half) + 32 * c;
          if constexpr (T::kTmaStore) {
            if (use_tma) {
              uint8_t* dst = stage_out + lane * 64;
              const int sw = (lane >> 1) & 3;
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 pk;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&h0);
                pk.y = *reinterpret_cast<uint32_t*>(&h1);
                pk.z = *reinterpret_cast<uint32_t*>(&h2);
                pk.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + ((i ^ sw) << 4)) = pk;
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tmap_c, stage_out_u32, ocol0 * 2, w.out_row_base + wrow0);
                bulk_commit_group();
              }
              continue;
            }
          }
          if (row_ok) {
            const long long o = w.out_off + static_cast<long long>(row) * p.ldc + ocol0;
            if constexpr (kOut == OUT_BF16) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (ocol0 + i < p.N) dst[i] = __float2bfloat16_rn(v[i]);
            } else {
              float* dst = reinterpret_cast<float*>(p.out) + o;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (ocol0 + i < p.N) dst[i] = v[i];
            }
          }
        }
      }
    }
    // the staging slots must not be released while a TMA store still reads them; the writes themselves are complete
    // at the end of the grid, and nothing in this kernel reads what they write
    if (lane == 0) bulk_wait_read_all();
  } else if (warp >= T::kUnpackWarp0) {
    // ------------------------------------------------------------------ unpack (int4 only)
    if constexpr (T::kRegBalance) {
      if constexpr (T::kUnpackRaises) reg_alloc<T::kRegsUnpack>();
      else reg_dealloc<T::kRegsUnpack>();
    }
    if constexpr (kTmemA) {
      // A through TMEM: the first four unpack warps own A, the other four B (below).  Warp w may touch TMEM lanes
      // 32 (w % 4) .. + 31, and lane = row of A: a thread expands the 64 packed bytes of ITS row of the K block
      // (four 16-byte loads from the staging tile, which TMA wrote with the 64-byte swizzle so that rows 64 bytes
      // apart do not collide on banks) into 32 words of int8 and stores them to the stage's 32 TMEM columns.
      // Packed chunk c (bytes 16c .. 16c+15) gives K slots 32c .. 32c+15 (low nibbles) and 32c+16 .. 32c+31 (high
      // nibbles), the same order the B operand uses; a 32-bit TMEM column holds four consecutive slots.
      if (warp < T::kUnpackWarp0 + 4) {
        const int row = (warp & 3) * 32 + lane;
        const uint32_t a_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t src_row = row * 64;
        const uint32_t sw = (row >> 1) & 3;
        int it = 0;
        bool ok = true;
        for (int t = tile0; t < num_tiles && ok; t += tile_step) {
          const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
          for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
            const int ps = it % PS;
            const uint32_t pph = (it / PS) & 1;
            const int s = it % S;
            const uint32_t ph = (it / S) & 1;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(pk_full_bar(ps), pph, ctx, 42))) { ok = false; break; }
            const uint8_t* pk_a = smem_gen + S * T::kStageBytes + ps * T::kPkStageBytes;
            uint4 x[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) x[c] = *reinterpret_cast<const uint4*>(pk_a + src_row + ((c ^ sw) << 4));
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty_bar(s), ph ^ 1u, ctx, 43))) { ok = false; break; }
            tc_fence_after_sync();
            uint32_t r[32];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              expand_word(x[c].x, r[8 * c + 0], r[8 * c + 4]);
              expand_word(x[c].y, r[8 * c + 1], r[8 * c + 5]);
              expand_word(x[c].z, r[8 * c + 2], r[8 * c + 6]);
              expand_word(x[c].w, r[8 * c + 3], r[8 * c + 7]);
            }
            tmem_st_32x32b_x32(tmem_base + a_lane + T::kTmemAStage0 + s * 32, r);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(full_bar(s));
              mbar_arrive(pk_empty_bar(ps));
            }
          }
        }
      }
    }
    if constexpr (kInt4) {
      if (!kTmemA || warp >= T::kUnpackWarp0 + 4) {
      constexpr int UT = kTmemA ? 128 : T::kUnpackWarps * 32;           // unpack threads of this role: 128 or 256
      const int ut = threadIdx.x - (T::kUnpackWarp0 + (kTmemA ? 4 : 0)) * 32;
      // Every item is one 16-byte load of packed data (32 nibbles) that becomes two 16-byte
      // chunks of int8.  Per-thread offsets are fixed; successive passes add a constant.
      //
      // A, K-major.  Packed tile [128 rows][64 B].  Item (r, c): row r, packed chunk c (0..3)
      // -> int8 chunks 2c (low nibbles) and 2c+1 (high nibbles) of row r, XOR-swizzled by r & 7.
      constexpr int kARowsPerPass = UT / 4;               // 32 or 64 (multiple of 8: r & 7 is fixed)
      const int a_r0 = ut >> 2, a_c = ut & 3;
      const uint32_t a_src0 = a_r0 * 64 + a_c * 16;
      const uint32_t a_row_off = (a_r0 >> 3) * 1024 + (a_r0 & 7) * 128;
      const uint32_t a_dst_lo0 = a_row_off + (((2 * a_c) ^ (a_r0 & 7)) << 4);
      const uint32_t a_dst_hi0 = a_row_off + (((2 * a_c + 1) ^ (a_r0 & 7)) << 4);
      // MN-major block of 128 columns.  Packed tile [64 K rows][128 B].  Item (pr, cn): packed
      // row pr -> K slots 32*(pr/16) + pr%16 (low) and +16 (high), chunk cn swizzled by slot & 7.
      constexpr int kMRowsPerPass = UT / 8;               // A (one block): 16 or 32 packed rows per pass
      const int m_p0 = ut >> 3, m_cn = ut & 7;
      const int m_slot0 = 32 * (m_p0 >> 4) + (m_p0 & 15);
      const uint32_t m_src0 = m_p0 * 128 + m_cn * 16;
      const uint32_t m_dst0 = m_slot0 * 128 + ((m_cn ^ (m_slot0 & 7)) << 4);
      constexpr int kBRowsPerPass = UT / 16;              // B (two blocks): 8 or 16 packed rows per pass
      const int b_p0 = ut >> 4, b_blk = (ut >> 3) & 1, b_cn = ut & 7;
      const uint32_t b_src0 = b_blk * (T::kPkBBytes / 2) + b_p0 * 128 + b_cn * 16;
      const uint32_t b_dst0 = b_blk * (T::kB8Bytes / 2) + b_p0 * 128 + ((b_cn ^ (b_p0 & 7)) << 4);
      int it = 0;
      bool ok = true;
      for (int t = tile0; t < num_tiles && ok; t += tile_step) {
        const TileWork w = decode_tile<kAMn, k2Cta, kTail, kWide>(p, t, cta_rank, unit);
        for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
          const int ps = it % PS;
          const uint32_t pph = (it / PS) & 1;
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(pk_full_bar(ps), pph, ctx, 40))) { ok = false; break; }
          const uint8_t* pk_a = smem_gen + S * T::kStageBytes + ps * T::kPkStageBytes;
          const uint8_t* pk_b = pk_a + T::kPkABytes;
          // all loads of the stage first: they do not depend on the int8 stage being free
          // B items are handled in batches of at most 4 to bound the registers holding raw data
          constexpr bool kOneB = T::kBBlocks == 1;
          constexpr int kBItems = (kOneB ? 512 : 1024) / UT;  // one or two 128-wide blocks of B
          constexpr int kBBatch = kBItems < 4 ? kBItems : 4;
          uint4 xa[kTmemA ? 1 : 512 / UT];
          uint4 xb[kBBatch];  // K-major B: packed tile [256 rows][64 B], same item scheme as K-major A
          auto load_b = [&](int j) -> uint4 {
            if constexpr (kBMn && kOneB) return *reinterpret_cast<const uint4*>(pk_b + m_src0 + j * (kMRowsPerPass * 128));
            else if constexpr (kBMn) return *reinterpret_cast<const uint4*>(pk_b + b_src0 + j * (kBRowsPerPass * 128));
            else return *reinterpret_cast<const uint4*>(pk_b + a_src0 + j * (kARowsPerPass * 64));
          };
          if constexpr (!kTmemA) {
#pragma unroll
            for (int j = 0; j < 512 / UT; ++j) {
              if constexpr (!kAMn) xa[j] = *reinterpret_cast<const uint4*>(pk_a + a_src0 + j * (kARowsPerPass * 64));
              else xa[j] = *reinterpret_cast<const uint4*>(pk_a + m_src0 + j * (kMRowsPerPass * 128));
            }
          }
#pragma unroll
          for (int j = 0; j < kBBatch; ++j) xb[j] = load_b(j);
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty_bar(s), ph ^ 1u, ctx, 41))) { ok = false; break; }
          uint8_t* a8 = smem_gen + s * T::kStageBytes;
          uint8_t* b8 = a8 + T::kA8Bytes;
#pragma unroll
          for (int j = 0; j < (kTmemA ? 0 : 512 / UT); ++j) {
            uint4 lo, hi;
            expand_word(xa[j].x, lo.x, hi.x);
            expand_word(xa[j].y, lo.y, hi.y);
            expand_word(xa[j].z, lo.z, hi.z);
            expand_word(xa[j].w, lo.w, hi.w);
            if constexpr (!kAMn) {
              *reinterpret_cast<uint4*>(a8 + a_dst_lo0 + j * (kARowsPerPass * 128)) = lo;
              *reinterpret_cast<uint4*>(a8 + a_dst_hi0 + j * (kARowsPerPass * 128)) = hi;
            } else {
              // packed rows advance by a multiple of 16 per pass: 32 K slots per 16 packed rows
              const uint32_t d = m_dst0 + j * ((kMRowsPerPass / 16) * 32 * 128);
              *reinterpret_cast<uint4*>(a8 + d) = lo;
              *reinterpret_cast<uint4*>(a8 + d + 16 * 128) = hi;
            }
          }
#pragma unroll
          for (int jb = 0; jb < kBItems; jb += kBBatch) {
#pragma unroll
            for (int jj = 0; jj < kBBatch; ++jj) {
              const int j = jb + jj;
              uint4 lo, hi;
              expand_word(xb[jj].x, lo.x, hi.x);
              expand_word(xb[jj].y, lo.y, hi.y);
              expand_word(xb[jj].z, lo.z, hi.z);
              expand_word(xb[jj].w, lo.w, hi.w);
              if (jb + kBBatch < kBItems) xb[jj] = load_b(j + kBBatch);  // next batch, in flight during the stores
              if constexpr (!kBMn) {
                if constexpr (kMaskK) {
                  // K-major B [N, K/2]: this thread's items all cover k = kb * 128 + 32 a_c .. + 31, byte j of `lo`
                  // holding k = ... + 2 j and byte j of `hi` k = ... + 2 j + 1: keep the bytes below the group's length
                  const int valid = w.k_valid - (kb * BK + 32 * a_c);
                  if (valid < 32) {
                    auto keep = [](uint4 x, int bytes) -> uint4 {
                      auto word = [&](uint32_t v, int first) -> uint32_t {
                        const int nb = bytes - first;
                        return nb >= 4 ? v : (nb <= 0 ? 0u : (v & ((1u << (8 * nb)) - 1u)));
                      };
                      return make_uint4(word(x.x, 0), word(x.y, 4), word(x.z, 8), word(x.w, 12));
                    };
                    lo = keep(lo, (valid + 1) >> 1);
                    hi = keep(hi, valid >> 1);
                  }
                }
                *reinterpret_cast<uint4*>(b8 + a_dst_lo0 + j * (kARowsPerPass * 128)) = lo;
                *reinterpret_cast<uint4*>(b8 + a_dst_hi0 + j * (kARowsPerPass * 128)) = hi;
              } else if constexpr (kOneB) {
                // one block, same item scheme as an MN-major A: packed row m_p0 + kMRowsPerPass * j
                if constexpr (kMaskK) {
                  const int k_lo = kb * BK + 2 * (m_p0 + kMRowsPerPass * j);
                  if (k_lo >= w.k_valid || k_lo < w.k_first) lo = make_uint4(0, 0, 0, 0);
                  if (k_lo + 1 >= w.k_valid) hi = make_uint4(0, 0, 0, 0);
                }
                const uint32_t d = m_dst0 + j * ((kMRowsPerPass / 16) * 32 * 128);
                *reinterpret_cast<uint4*>(b8 + d) = lo;
                *reinterpret_cast<uint4*>(b8 + d + 16 * 128) = hi;
              } else {
                // packed row of this pass: b_p0 + kBRowsPerPass * j  (b_p0 < kBRowsPerPass <= 16)
                constexpr int R = kBRowsPerPass;
                const int row_adv = R * j;                       // compile-time after unrolling
                const int slot_adv = 32 * (row_adv >> 4) + (row_adv & 15);
                if constexpr (kMaskK) {
                  const int k_lo = kb * BK + 2 * (b_p0 + row_adv);
                  if (k_lo >= w.k_valid || k_lo < w.k_first) lo = make_uint4(0, 0, 0, 0);
                  if (k_lo + 1 >= w.k_valid) hi = make_uint4(0, 0, 0, 0);
                }
                const uint32_t d = b_dst0 + slot_adv * 128;
                *reinterpret_cast<uint4*>(b8 + d) = lo;
                *reinterpret_cast<uint4*>(b8 + d + 16 * 128) = hi;
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(full_bar(s));
            mbar_arrive(pk_empty_bar(ps));
          }
        }
      }
      }  // B role (or the only unpack role)
    }
  }

  // ------------------------------------------------------------------ teardown
  // After a wait ran out some role may have left copies or MMAs in flight that target this CTA's shared
  // memory or TMEM: give them time to land (they take microseconds) before the CTA's resources are released.
  if (*abort_flag != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < ABORT_DRAIN_NS) {
    }
  }
  tc_fence_before_sync();
  if constexpr (k2Cta) cluster_sync_all();  // the peer no longer touches this CTA's shared memory or TMEM
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (k2Cta) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace b200
