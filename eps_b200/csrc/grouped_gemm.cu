// FP8 (e4m3) block-scaled grouped GEMM for sm_100a: tcgen05.mma + TMEM + TMA.
//
// Replaces the reference's sm_90 CUTLASS grouped GEMM (src/gemm/aok_grouped_gemm/
// src/operations/hopper_grouped_gemm_kernel.h:228-400) and, through its epilogues,
// silu_activate (src/executor/activations.cu:9-40) and the weight multiply of
// localReduce (src/scheduler/local_reducer.cu:137).
//
// Shape of the kernel
//   * persistent: one CTA per SM walks tiles t = blockIdx.x, += gridDim.x of a
//     ragged tile list built on the device from the expert prefix sum;
//   * tile = 128 rows (tokens) x 256 weight rows, K step 128 (= one 128-byte
//     swizzle atom of e4m3, four tcgen05.mma of K=32);
//   * warp 0 issues TMA loads into a 3-stage shared-memory ring, warps 1 and 2 issue
//     the MMAs of the even / odd K steps into one of two 256-column TMEM buffers, warps 4..11 (two
//     warpgroups) drain a TMEM buffer per K step with tcgen05.ld and fold it
//     into fp32 register accumulators multiplied by a_scale[row,kb]*b_scale[nb,kb]
//     (the scales are plain fp32, so the hardware's power-of-two block scaling
//     cannot be used and the promotion is done on the CUDA cores);
//   * every wait on an mbarrier is bounded: after ~2 s it records a code in the
//     caller's status words, raises a CTA-wide abort flag, and every role leaves
//     its loop, waits for copies in flight, frees TMEM and returns.
//   * an m-tile with at most 64 valid rows (an expert's remainder past a multiple of 128, or a small expert) is
//     computed with the operand roles swapped, from the same shared-memory stage: its two 128-row weight blocks
//     are the M of two MMAs and its 32 or 64 token rows their N, so its drain costs in proportion to the tokens;
//   * no TMA multicast is used anywhere.
#include <atomic>

#include "tc_ptx.cuh"

namespace epsb {

namespace {

constexpr int kBM = 128;           // rows per tile
constexpr int kBN = 256;           // weight rows per tile (two 128-row TMA boxes)
constexpr int kBK = 128;           // K step (bytes == elements for e4m3)
// Shared memory is split between the TMA ring and the staging rows of the tile output.  Gate/up stores 64 bytes per
// thread and keeps four stages (measured: 5.6 vs 5.2 TB/s of weight streaming at 128 rows per expert); the bf16 modes
// store 256 bytes per thread and keep three (their output staging is worth more than the fourth stage).
template <int kMode>
struct ModeCfg {
  static constexpr int kStages = kMode == EPSB_GEMM_GATEUP ? 4 : 3;
  static constexpr int kOutRowBytes = (kMode == EPSB_GEMM_GATEUP ? 64 : 256) + 16;  // + padding against bank conflicts
};
constexpr int kABytes = kBM * kBK;         // 16 KB
constexpr int kBBytes = kBN * kBK;         // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 384;              // warpgroup 0: producers; warpgroups 1,2: epilogue
constexpr int kTmemCols = 512;             // two accumulator buffers of 256 fp32 columns
constexpr int kMaxExperts = 1024;

constexpr uint32_t kIdesc = f8_idesc(kBM, kBN);

template <int kMode>
struct SharedStorage {
  static constexpr int kStages = ModeCfg<kMode>::kStages;
  static constexpr int kOutRowBytes = ModeCfg<kMode>::kOutRowBytes;
  // tile ring first: every stage base must be 1024-byte aligned for the 128-byte swizzle
  uint8_t tiles[kStages][kStageBytes];
  uint8_t out_stage[2][kBM][kOutRowBytes];  // [column half][row]: tile output on its way to global memory
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_empty[2];
  uint64_t amax_bar;
  uint32_t tmem_base;
  volatile int abort_flag;
  float amax_x[2][2][kBM];  // [tile parity][column half][row]
  int32_t tile_prefix[kMaxExperts + 1];  // m-tiles before each expert
};

struct GemmParams {
  const int32_t* a_rows;  // optional: GEMM row m reads row a_rows[m] of A and a_s (index-driven A loads)
  const float* a_s;
  const float* b_s;
  const int32_t* excl;
  void* C;
  float* c_s;
  const float* row_w;
  int32_t* status;
  int num_experts;
  int64_t max_rows;
  int64_t N;   // weight rows per expert (2I in gate/up mode)
  int64_t K;
  int n_tiles; // tiles along N per m-tile
};

struct TileCoord {
  int e, row0, rows_left, n;  // expert, first GEMM row of the tile, valid rows from row0, n-tile index
  int tail;                   // 0: token rows on the MMA's M; 32 or 64: a tail tile of that many token COLUMNS
};

// An m-tile with at most kTailMax valid rows (an expert's remainder, or a small expert) is computed with the
// operand roles swapped: the 2 x 128 weight rows of the tile become two M=128 MMAs and the tokens their N
// (32 or 64 columns), from the very same shared-memory stage.  Draining TMEM then costs in proportion to the
// tokens, where the normal orientation drains all 128 x 256 accumulators for a handful of valid rows.
constexpr int kTailMax = 64;

template <class Storage>
__device__ __forceinline__ TileCoord locate_tile(int t, const GemmParams& p, const Storage* sm) {
  const int g = t / p.n_tiles;
  TileCoord c;
  c.n = t - g * p.n_tiles;
  int lo = 0, hi = p.num_experts;  // find e with prefix[e] <= g < prefix[e+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sm->tile_prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  c.e = lo;
  const int m = g - sm->tile_prefix[lo];
  const int b = __ldg(p.excl + lo), e_ = __ldg(p.excl + lo + 1);
  c.row0 = b + m * kBM;
  c.rows_left = e_ - c.row0;
  c.tail = c.rows_left <= 32 ? 32 : (c.rows_left <= kTailMax ? 64 : 0);
  return c;
}

// Epilogue of a tail tile (see kTailMax).  TMEM lanes = the 128 weight rows of a block, columns [0, T) = block 0
// (gate rows, or the tile's first 128 weight rows), [T, 2T) = block 1 (up rows, or the second 128), T = 2 * kTh.
// The warp of quadrant `quad` and column half `half` owns weight rows 32*quad + lane and tokens
// [half*kTh, (half+1)*kTh) of the tile.  Token scales live one per lane and are broadcast with shuffles.
template <int kMode, int kTh, class Storage>
__device__ __forceinline__ bool tail_tile(const GemmParams& p, Storage* sm, const TileCoord& c, int KB, uint32_t& it,
                                          uint32_t& amax_phase, uint32_t lane_addr, int quad, int half, int lane) {
  constexpr int kT = 2 * kTh;
  const int NB = (int)(p.N / 128);
  const int tok0 = half * kTh;                           // first token (tile-relative) of this warp
  const bool tok_ok = lane < kTh && tok0 + lane < c.rows_left;
  const int64_t my_row = (int64_t)c.row0 + tok0 + lane;  // the token whose scale this lane carries
  const int64_t src_row = tok_ok ? my_row : (int64_t)c.row0;   // row of A / a_s this lane's token comes from
  const float* as_row = p.a_s + (p.a_rows != nullptr ? (int64_t)__ldg(p.a_rows + src_row) : src_row) * KB;
  int blk0, blk1;
  if (kMode == EPSB_GEMM_GATEUP) {
    blk0 = c.n;
    blk1 = NB / 2 + c.n;
  } else {
    blk0 = c.n * 2;
    blk1 = min(c.n * 2 + 1, NB - 1);
  }
  const float* bs0 = p.b_s + ((int64_t)c.e * NB + blk0) * KB;
  const float* bs1 = p.b_s + ((int64_t)c.e * NB + blk1) * KB;
  float acc0[kTh], acc1[kTh];
#pragma unroll
  for (int i = 0; i < kTh; i++) acc0[i] = acc1[i] = 0.0f;
  float sa = tok_ok ? __ldg(as_row) : 0.0f, sb0 = __ldg(bs0), sb1 = __ldg(bs1);
  for (int kb = 0; kb < KB; kb++, it++) {
    const float s0 = sa * sb0, s1 = sa * sb1;   // this lane's token, both weight blocks
    if (kb + 1 < KB) {
      sa = tok_ok ? __ldg(as_row + kb + 1) : 0.0f;
      sb0 = __ldg(bs0 + kb + 1);
      sb1 = __ldg(bs1 + kb + 1);
    }
    bool good = mbar_wait(&sm->empty[it % Storage::kStages], (it / Storage::kStages) & 1u, sm, p.status, 33);
    good = __all_sync(0xffffffffu, good);
    if (!good) return false;
    tc_fence_after();
    const uint32_t tb = lane_addr + (it & 1u) * (uint32_t)kBN + (uint32_t)tok0;
    uint32_t v0[kTh], v1[kTh];
    if constexpr (kTh == 16) {
      tmem_ld16_async(tb, v0);
      tmem_ld16_async(tb + kT, v1);
      tmem_wait16(v0);
      tmem_tie16(v1);
    } else {
      tmem_ld32_async(tb, v0);
      tmem_ld32_async(tb + kT, v1);
      tmem_wait(v0);
      tmem_tie(v1);
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->tmem_empty[it & 1u]);
#pragma unroll
    for (int i = 0; i < kTh; i++) {
      acc0[i] = fmaf(__uint_as_float(v0[i]), __shfl_sync(0xffffffffu, s0, i), acc0[i]);
      acc1[i] = fmaf(__uint_as_float(v1[i]), __shfl_sync(0xffffffffu, s1, i), acc1[i]);
    }
  }

  const int wr = quad * 32 + lane;  // weight row inside a 128-row block
  if (kMode == EPSB_GEMM_GATEUP) {
    const int64_t I = p.N / 2;
    // [tile parity][half][quadrant][token]: the same 512 floats the other orientation uses as [parity][half][row]
    float* ax = &sm->amax_x[0][0][0] + ((amax_phase * 2 + half) * 4) * 32;
#pragma unroll
    for (int i = 0; i < kTh; i++) {
      const float g = acc0[i], u = acc1[i];
      const float a = (g * __frcp_rn(1.0f + __expf(-g))) * u;
      acc0[i] = a;
      // |a| of a finite float orders like its bit pattern; a NaN (only in token columns past the expert's
      // rows, never stored) may win the maximum there and nowhere else
      const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(a)));
      if (lane == i) ax[quad * 32 + i] = __uint_as_float(m);
    }
    mbar_arrive(&sm->amax_bar);
    bool good = mbar_wait(&sm->amax_bar, amax_phase, sm, p.status, 43);
    good = __all_sync(0xffffffffu, good);
    if (!good) return false;
    float amax = 0.0f;
    if (lane < kTh) amax = fmaxf(fmaxf(ax[lane], ax[32 + lane]), fmaxf(ax[64 + lane], ax[96 + lane]));
    amax_phase ^= 1;
    const float scale = __fdiv_rn(amax, kFp8Max);
    const float inv = __frcp_rn(scale);
    uint8_t* q_out = reinterpret_cast<uint8_t*>(p.C) + ((int64_t)c.row0 + tok0) * I + (int64_t)c.n * 128 + wr;
#pragma unroll
    for (int i = 0; i < kTh; i++) {
      const float inv_i = __shfl_sync(0xffffffffu, inv, i);
      if (tok0 + i < c.rows_left)
        q_out[(int64_t)i * I] = (uint8_t)(cvt_e4m3x2(quant_clamp(acc0[i], inv_i), 0.0f) & 0xffu);
    }
    if (quad == 0 && tok_ok) p.c_s[my_row * (I / 128) + c.n] = scale;
  } else {
    float wgt = 1.0f;
    if (kMode == EPSB_GEMM_DOWN && p.row_w != nullptr && tok_ok) wgt = __ldg(p.row_w + my_row);
    const int64_t col0 = (int64_t)c.n * kBN + wr;
    const bool blk1_ok = (int64_t)c.n * kBN + 128 < p.N;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + ((int64_t)c.row0 + tok0) * p.N + col0;
#pragma unroll
    for (int i = 0; i < kTh; i++) {
      const float w = __shfl_sync(0xffffffffu, wgt, i);
      if (tok0 + i < c.rows_left) {
        out[(int64_t)i * p.N] = __float2bfloat16_rn(acc0[i] * w);
        if (blk1_ok) out[(int64_t)i * p.N + 128] = __float2bfloat16_rn(acc1[i] * w);
      }
    }
  }
  return true;
}

// Tensor maps of the activation matrix: a box of 128 rows for the normal tiles and boxes of 64 and 32 rows for
// tail tiles, which then fill 8 or 4 KB of the stage's A region instead of 16.
struct AMaps {
  CUtensorMap rows128, rows64, rows32;
  CUtensorMap row1;   // box of ONE row: the shape tile::gather4 loads take (four such rows per instruction)
};

// Four rows of A, picked by index, land as four consecutive 128-byte rows of the stage (TMA tile::gather4).  The
// 128-byte swizzle is a function of the shared-memory address, so 32 such loads fill the A region exactly like
// one 128-row box load would.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* map, int x, int r0, int r1, int r2, int r3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}

template <int kMode>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ AMaps tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  using Storage = SharedStorage<kMode>;
  constexpr int kStages = Storage::kStages;
  Storage* sm = reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (int)(p.K / kBK);

  // ---- set-up: barriers, TMEM, tile list
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&sm->tmem_empty[b], 8);  // one arrival per epilogue warp
    }
    mbar_init(&sm->amax_bar, 256);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp == 2) {
    // m-tiles before each expert: warp-wide scan, 32 experts per step
    int carry = 0;
    for (int e0 = 0; e0 < p.num_experts; e0 += 32) {
      const int e = e0 + lane;
      int mt = 0;
      if (e < p.num_experts) mt = (__ldg(p.excl + e + 1) - __ldg(p.excl + e) + kBM - 1) / kBM;
      int inc = mt;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += n;
      }
      if (e < p.num_experts) sm->tile_prefix[e] = carry + inc - mt;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) sm->tile_prefix[p.num_experts] = carry;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  const int total_tiles = sm->tile_prefix[p.num_experts] * p.n_tiles;

  // Register budget.  The CTA owns kThreads * 168 registers (what __launch_bounds__(384, 1) compiles to);
  // setmaxnreg.inc BLOCKS until the CTA's own pool can serve it, so the two numbers below must satisfy
  // 128 * dec + 256 * inc <= 384 * 168 = 64512, or the kernel hangs outside every bounded wait.
  static_assert(128 * 40 + 256 * 232 <= kThreads * 168, "setmaxnreg budget exceeds the CTA's register pool");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ------------------------------------------------ TMA producer.  Lane 0 waits for the stage, announces the
      // bytes and loads the weights; the A tile comes either as one box load (lane 0) or, when the caller gave a
      // row index per GEMM row, as one gather4 per lane (lane j brings tile rows 4j .. 4j+3).
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord c = locate_tile(t, p, sm);
        int brow0, brow1;  // first weight row of each 128-row box
        if (kMode == EPSB_GEMM_GATEUP) {
          brow0 = (int)(c.e * p.N + c.n * 128);
          brow1 = (int)(c.e * p.N + p.N / 2 + c.n * 128);
        } else {
          brow0 = (int)(c.e * p.N + c.n * kBN);
          brow1 = brow0 + 128;
        }
        const int a_rows_tile = c.tail ? c.tail : kBM;   // rows of A this tile stages
        int r4[4] = {0, 0, 0, 0};
        if (p.a_rows != nullptr) {
          // rows past the expert's end repeat its first row: loaded, multiplied, never stored
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const int r = 4 * lane + i;
            r4[i] = __ldg(p.a_rows + c.row0 + (r < c.rows_left ? r : 0));
          }
        }
        for (int kb = 0; kb < KB; kb++, it++) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (lane == 0) ok = mbar_wait(&sm->empty[s], ph ^ 1, sm, p.status, 11);
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          if (!ok) break;
          uint8_t* base = sm->tiles[s];
          if (lane == 0) {
            mbar_expect_tx(&sm->full[s], a_rows_tile * kBK + kBBytes);
            if (p.a_rows == nullptr)
              tma_load_2d(base, c.tail == 0 ? &tmap_a.rows128 : (c.tail == 64 ? &tmap_a.rows64 : &tmap_a.rows32), kb * kBK,
                          c.row0, &sm->full[s]);
            tma_load_2d(base + kABytes, &tmap_b, kb * kBK, brow0, &sm->full[s]);
            tma_load_2d(base + kABytes + kABytes, &tmap_b, kb * kBK, brow1, &sm->full[s]);
          }
          if (p.a_rows != nullptr && 4 * lane < a_rows_tile)
            tma_gather4(base + lane * 4 * kBK, &tmap_a.row1, kb * kBK, r4[0], r4[1], r4[2], r4[3], &sm->full[s]);
        }
      }
      if (!ok && lane == 0) {
        // let copies already issued land before the CTA's shared memory is released
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ------------------------------------------------ MMA issuers: warp 1 takes the even K steps (accumulator
      // buffer 0), warp 2 the odd ones (buffer 1).  A K step's MMAs accumulate from scratch into their own buffer, so
      // the two threads need no order between them.  One thread alone cannot keep the tensor pipe fed: its chain per
      // K step (wait for the buffer, wait for the stage, four MMAs whose issue is paced by the pipe, two commits) has
      // ~500 cycles of barrier latency in it during which nothing is queued behind the MMAs in flight; with two
      // threads the waits of step it+1 run while the MMAs of step it execute.
      const uint32_t me = (uint32_t)(warp - 1);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int tail = locate_tile(t, p, sm).tail;
        const uint32_t idesc_tail = f8_idesc(128, tail);
        for (int kb = 0; kb < KB; kb++, it++) {
          if ((it & 1u) != me) continue;
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          const int buf = it & 1;
          const uint32_t tph = (it >> 1) & 1;
          if (!(ok = mbar_wait(&sm->tmem_empty[buf], tph ^ 1, sm, p.status, 21))) break;
          if (!(ok = mbar_wait(&sm->full[s], ph, sm, p.status, 22))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sm->tiles[s]);
          const uint64_t da = ((uint64_t)kDescHi << 32) | (uint64_t)(((a_addr >> 4) & 0x3fffu) | (1u << 16));
          const uint64_t db = ((uint64_t)kDescHi << 32) | (uint64_t)((((a_addr + kABytes) >> 4) & 0x3fffu) | (1u << 16));
          const uint32_t d = tmem_base + (uint32_t)buf * kBN;
          if (tail == 0) {
#pragma unroll
            for (int k4 = 0; k4 < kBK / 32; k4++) umma_f8(d, da + 2 * k4, db + 2 * k4, kIdesc, k4 > 0 ? 1u : 0u);
          } else {
            // weights on M (two 128-row blocks of the stage's B region), the tile's token rows on N
            const uint64_t dw1 =
                ((uint64_t)kDescHi << 32) | (uint64_t)((((a_addr + 2 * kABytes) >> 4) & 0x3fffu) | (1u << 16));
#pragma unroll
            for (int k4 = 0; k4 < kBK / 32; k4++) {
              umma_f8(d, db + 2 * k4, da + 2 * k4, idesc_tail, k4 > 0 ? 1u : 0u);
              umma_f8(d + (uint32_t)tail, dw1 + 2 * k4, da + 2 * k4, idesc_tail, k4 > 0 ? 1u : 0u);
            }
          }
          // ONE commit per K step: when these MMAs have completed the stage may be refilled (the producer waits on
          // this barrier) and the accumulator buffer is ready (the epilogue warps wait on the same barrier)
          umma_commit(&sm->empty[s]);
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ------------------------------------------------ epilogue: 8 warps
    const int ew = warp - 4;           // 0..7
    const int quad = warp & 3;         // TMEM lane quadrant this warp may read
    const int half = ew >> 2;          // which half of the tile's columns
    const int r_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int KBs = KB;                // scales per row
    const int NB = (int)(p.N / 128);
    uint32_t it = 0, amax_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const TileCoord c = locate_tile(t, p, sm);
      if (c.tail != 0) {
        ok = c.tail == 32 ? tail_tile<kMode, 16>(p, sm, c, KB, it, amax_phase, lane_addr, quad, half, lane)
                          : tail_tile<kMode, 32>(p, sm, c, KB, it, amax_phase, lane_addr, quad, half, lane);
        continue;
      }
      const int64_t grow = (int64_t)c.row0 + r_in_tile;
      const bool row_ok = r_in_tile < c.rows_left;
      const int64_t src_row = row_ok ? grow : (int64_t)c.row0;
      const float* as_row = p.a_s + (p.a_rows != nullptr ? (int64_t)__ldg(p.a_rows + src_row) : src_row) * KBs;
      // the two 128-wide scale blocks this thread's columns belong to
      const float* bs0;
      const float* bs1;
      if (kMode == EPSB_GEMM_GATEUP) {
        bs0 = p.b_s + ((int64_t)c.e * NB + c.n) * KBs;               // gate block
        bs1 = p.b_s + ((int64_t)c.e * NB + NB / 2 + c.n) * KBs;      // up block
      } else {
        bs0 = p.b_s + ((int64_t)c.e * NB + min(c.n * 2 + half, NB - 1)) * KBs;
        bs1 = bs0;
      }
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; i++) acc[i] = 0.0f;
      float sa = __ldg(as_row), sb0 = __ldg(bs0), sb1 = __ldg(bs1);
      float s0 = 0.0f, s1 = 0.0f;
      // gate/up mode: chunks 0,1 = gate columns [64*half, +64), chunks 2,3 = up columns [128+64*half, +64)
      auto col_of = [&](int ch) -> uint32_t {
        if (kMode == EPSB_GEMM_GATEUP) return (uint32_t)((ch < 2 ? 0 : 128) + 64 * half + (ch & 1) * 32);
        return (uint32_t)(128 * half + ch * 32);
      };
      auto tmem_of = [&](uint32_t k_it) -> uint32_t { return lane_addr + (k_it & 1u) * (uint32_t)kBN; };
      auto wait_full = [&](uint32_t k_it) -> bool {
        bool good = mbar_wait(&sm->empty[k_it % kStages], (k_it / kStages) & 1u, sm, p.status, 31);
        good = __all_sync(0xffffffffu, good);
        if (good) tc_fence_after();
        return good;
      };
      // Drain of a K step, software-pipelined: the thread's 128 columns leave TMEM as four loads of 32 columns,
      // and the load of chunk c+1 is issued BEFORE the fold of chunk c, so that TMEM reads and FMAs of one warp
      // overlap (tcgen05.wait::ld waits for every load the thread has in flight, hence exactly one is kept in
      // flight).  The chain crosses K steps: once the fourth load of a step has landed the buffer is released to
      // the MMA warp, the first load of the NEXT step is issued, and only then is the fourth chunk folded.
      // Two 32-register landing arrays beside the 128 accumulators: no spills at 232 registers.
      uint32_t t0[32], t1[32];
      ok = wait_full(it);
      if (!ok) break;
      tmem_ld32_async(tmem_of(it) + col_of(0), t0);
      for (int kb = 0; kb < KB; kb++, it++) {
        s0 = sa * sb0;
        s1 = sa * sb1;
        if (kb + 1 < KB) {
          sa = __ldg(as_row + kb + 1);
          sb0 = __ldg(bs0 + kb + 1);
          sb1 = __ldg(bs1 + kb + 1);
        }
        const float sc = kMode == EPSB_GEMM_GATEUP ? s1 : s0;
        const uint32_t tb = tmem_of(it);
        tmem_wait(t0);
        tmem_ld32_async(tb + col_of(1), t1);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[i] = fmaf(__uint_as_float(t0[i]), s0, acc[i]);
        tmem_wait(t1);
        tmem_ld32_async(tb + col_of(2), t0);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[32 + i] = fmaf(__uint_as_float(t1[i]), s0, acc[32 + i]);
        tmem_wait(t0);
        tmem_ld32_async(tb + col_of(3), t1);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[64 + i] = fmaf(__uint_as_float(t0[i]), sc, acc[64 + i]);
        tmem_wait(t1);   // every load of this K step has landed: the buffer may be overwritten
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->tmem_empty[it & 1u]);
        if (kb + 1 < KB) {
          ok = wait_full(it + 1);
          if (!ok) break;
          tmem_ld32_async(tmem_of(it + 1) + col_of(0), t0);
        }
#pragma unroll
        for (int i = 0; i < 32; i++) acc[96 + i] = fmaf(__uint_as_float(t1[i]), sc, acc[96 + i]);
      }
      if (!ok) break;

      // ---- tile epilogue
      if (kMode == EPSB_GEMM_GATEUP) {
        const int64_t I = p.N / 2;
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 64; i++) {
          const float g = acc[i], u = acc[64 + i];
          const float a = (g * __frcp_rn(1.0f + __expf(-g))) * u;  // silu(g) * u; checked by tolerance, not bit-exact
          acc[i] = a;
          amax = fmaxf(amax, fabsf(a));
        }
        sm->amax_x[amax_phase][half][r_in_tile] = amax;
        mbar_arrive(&sm->amax_bar);
        ok = mbar_wait(&sm->amax_bar, amax_phase, sm, p.status, 41);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        amax = fmaxf(amax, sm->amax_x[amax_phase][half ^ 1][r_in_tile]);
        amax_phase ^= 1;
        const float scale = __fdiv_rn(amax, kFp8Max);
        const float inv = __frcp_rn(scale);
        uint8_t* stage_row = sm->out_stage[half][r_in_tile];
        bulk_wait_read();  // this thread's copy of the previous tile has left the staging row
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int i = q4 * 16 + j * 4;
              w[j] = (uint32_t)cvt_e4m3x2(quant_clamp(acc[i], inv), quant_clamp(acc[i + 1], inv)) |
                     ((uint32_t)cvt_e4m3x2(quant_clamp(acc[i + 2], inv), quant_clamp(acc[i + 3], inv)) << 16);
            }
            st_shared_16(stage_row + q4 * 16, make_uint4(w[0], w[1], w[2], w[3]));
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          bulk_store_row(reinterpret_cast<uint8_t*>(p.C) + grow * I + (int64_t)c.n * 128 + 64 * half, stage_row, 64);
          bulk_commit();
          if (half == 0) p.c_s[grow * (I / 128) + c.n] = scale;
        }
        // amax_x alternates between two copies: a copy is rewritten two tiles later, and a thread
        // cannot pass the next tile's amax_bar before its partner has arrived there, i.e. has read.
      } else {
        const int64_t col0 = (int64_t)c.n * kBN + 128 * half;
        uint8_t* stage_row = sm->out_stage[half][r_in_tile];
        bulk_wait_read();  // this thread's copy of the previous tile has left the staging row
        if (row_ok && col0 < p.N) {
          float wgt = 1.0f;
          if (kMode == EPSB_GEMM_DOWN && p.row_w != nullptr) wgt = __ldg(p.row_w + grow);
          // The thread's 256 bytes go to its own padded row of shared memory (16-byte stores of a warp land in
          // distinct banks) and leave for global memory as ONE asynchronous 256-byte bulk copy, instead of sixteen
          // scattered 16-byte stores per thread; the copy overlaps the next tile's K loop.
#pragma unroll
          for (int q8 = 0; q8 < 16; q8++) {
            uint4 o;
            o.x = pack_bf16x2(acc[q8 * 8 + 0] * wgt, acc[q8 * 8 + 1] * wgt);
            o.y = pack_bf16x2(acc[q8 * 8 + 2] * wgt, acc[q8 * 8 + 3] * wgt);
            o.z = pack_bf16x2(acc[q8 * 8 + 4] * wgt, acc[q8 * 8 + 5] * wgt);
            o.w = pack_bf16x2(acc[q8 * 8 + 6] * wgt, acc[q8 * 8 + 7] * wgt);
            st_shared_16(stage_row + q8 * 16, o);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          bulk_store_row(reinterpret_cast<uint8_t*>(p.C) + (grow * p.N + col0) * 2, stage_row, 256);
          bulk_commit();
        }
      }
    }
    bulk_wait_all();  // every staged row has reached global memory before the CTA's shared memory goes away
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------- host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

// 2-D e4m3 tensor [rows, K] (K contiguous), box 128 bytes x box_rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows = 128) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(EPSB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EPSB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return EPSB_OK;
}

template <int kMode>
int launch(const AMaps& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  const size_t smem = sizeof(SharedStorage<kMode>) + 1024;
  // the attribute belongs to the (kernel, device) pair: set it once per device
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaFuncSetAttribute(gemm): %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  grouped_gemm_fp8_kernel<kMode><<<grid, kThreads, smem, st>>>(ta, tb, p);
  return check_launch("grouped_gemm_fp8");
}

}  // namespace

}  // namespace epsb

using namespace epsb;

// a_rows == nullptr: GEMM row m is row m of A (a_src_rows = max_rows).  Otherwise GEMM row m is row a_rows[m] of the
// a_src_rows x K matrix A (and of a_s).
static int grouped_gemm_fp8_impl(int mode, const void* A, const float* a_s, int64_t a_src_rows, const int32_t* a_rows,
                                 const void* B, const float* b_s, const int32_t* excl, int num_experts, int64_t max_rows,
                                 int64_t N, int64_t K, void* C, float* c_s, const float* row_w, int32_t* status,
                                 int sm_count, void* stream) {
  EPSB_REQUIRE(sm_count >= 0, EPSB_ERR_INVALID, "sm_count %d is negative", sm_count);
  EPSB_REQUIRE(mode == EPSB_GEMM_PLAIN || mode == EPSB_GEMM_GATEUP || mode == EPSB_GEMM_DOWN, EPSB_ERR_INVALID,
               "unknown GEMM mode %d", mode);
  EPSB_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts, EPSB_ERR_INVALID, "num_experts %d out of range",
               num_experts);
  EPSB_REQUIRE(K > 0 && K % 128 == 0, EPSB_ERR_INVALID, "K: %lld is not divisible by 128", (long long)K);
  EPSB_REQUIRE(N > 0 && N % 128 == 0, EPSB_ERR_INVALID, "N: %lld is not divisible by 128", (long long)N);
  EPSB_REQUIRE(mode != EPSB_GEMM_GATEUP || (N % 256 == 0 && c_s != nullptr), EPSB_ERR_INVALID,
               "gate/up mode needs N = 2*I with I %% 128 == 0 and an output scale buffer");
  EPSB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0, EPSB_ERR_INVALID,
               "A, B and C must be 16-byte aligned");
  EPSB_REQUIRE((int64_t)num_experts * N < (1ll << 31) && max_rows < (1ll << 31) && a_src_rows < (1ll << 31),
               EPSB_ERR_INVALID, "tensor too large for 32-bit TMA coordinates");
  if (max_rows <= 0) return EPSB_OK;
  EPSB_REQUIRE(a_src_rows > 0, EPSB_ERR_INVALID, "the source matrix of A has no rows");
  AMaps ta;
  CUtensorMap tb;
  int rc = make_map(&ta.rows128, A, a_src_rows, K, 128);
  if (rc) return rc;
  rc = make_map(&ta.rows64, A, a_src_rows, K, 64);
  if (rc) return rc;
  rc = make_map(&ta.rows32, A, a_src_rows, K, 32);
  if (rc) return rc;
  rc = make_map(&ta.row1, A, a_src_rows, K, 1);
  if (rc) return rc;
  rc = make_map(&tb, B, (int64_t)num_experts * N, K);
  if (rc) return rc;
  GemmParams p;
  p.a_rows = a_rows;
  p.a_s = a_s;
  p.b_s = b_s;
  p.excl = excl;
  p.C = C;
  p.c_s = c_s;
  p.row_w = row_w;
  p.status = status;
  p.num_experts = num_experts;
  p.max_rows = max_rows;
  p.N = N;
  p.K = K;
  p.n_tiles = mode == EPSB_GEMM_GATEUP ? (int)(N / 256) : (int)((N + kBN - 1) / kBN);
  // tile-count upper bound without reading the device-side prefix sum
  const int64_t m_tiles_max = (max_rows + kBM - 1) / kBM + num_experts;
  int64_t grid = m_tiles_max * p.n_tiles;
  if (grid > gemm_cta_limit(sm_count)) grid = gemm_cta_limit(sm_count);
  auto st = static_cast<cudaStream_t>(stream);
  switch (mode) {
    case EPSB_GEMM_GATEUP: return launch<EPSB_GEMM_GATEUP>(ta, tb, p, (int)grid, st);
    case EPSB_GEMM_DOWN: return launch<EPSB_GEMM_DOWN>(ta, tb, p, (int)grid, st);
    default: return launch<EPSB_GEMM_PLAIN>(ta, tb, p, (int)grid, st);
  }
}

extern "C" int epsb_grouped_gemm_fp8(int mode, const void* A, const float* a_s, const void* B, const float* b_s,
                                     const int32_t* excl, int num_experts, int64_t max_rows, int64_t N, int64_t K,
                                     void* C, float* c_s, const float* row_w, int32_t* status, int sm_count,
                                     void* stream) {
  return grouped_gemm_fp8_impl(mode, A, a_s, max_rows, nullptr, B, b_s, excl, num_experts, max_rows, N, K, C, c_s, row_w,
                               status, sm_count, stream);
}

extern "C" int epsb_grouped_gemm_fp8_gather(int mode, const void* A_src, const float* a_s_src, int64_t a_src_rows,
                                            const int32_t* a_rows, const void* B, const float* b_s, const int32_t* excl,
                                            int num_experts, int64_t max_rows, int64_t N, int64_t K, void* C, float* c_s,
                                            const float* row_w, int32_t* status, int sm_count, void* stream) {
  EPSB_REQUIRE(a_rows != nullptr, EPSB_ERR_INVALID, "a_rows is NULL: use epsb_grouped_gemm_fp8");
  return grouped_gemm_fp8_impl(mode, A_src, a_s_src, a_src_rows, a_rows, B, b_s, excl, num_experts, max_rows, N, K, C,
                               c_s, row_w, status, sm_count, stream);
}
