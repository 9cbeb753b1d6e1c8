// bf16 x bf16 -> bf16 grouped GEMM for sm_100a (tcgen05.mma kind::f16 + TMEM + TMA): the reference's own GEMM op.
//
// Replaces AokGroupedGemm::run -> SM90_GROUPED_GEMM::Launch (src/executor/aok_grouped_gemm.cu:22-37,
// src/gemm/aok_grouped_gemm/src/operations/hopper_grouped_gemm_kernel.h:228-400): for local expert e, rows
// [excl[e], excl[e+1]) of A times B[e]^T, alpha = 1, beta = 0, fp32 accumulation, one rounding to bf16.
//
// Shape of the kernel: persistent, one CTA per SM over a ragged tile list built on the device from the expert prefix
// sum (never read on the host); tile = 128 rows x 256 weight rows; K block = 64 elements (one 128-byte swizzle
// atom of bf16, four MMAs of K=16).  Warp 0 issues TMA loads into a 3-stage ring, warp 1 issues the MMAs, which
// accumulate over the WHOLE K extent in one of two 256-column TMEM buffers (no per-K-block drain: there are no
// block scales here), warps 4..11 drain a finished buffer while the next tile accumulates in the other one,
// stage their bf16 rows in shared memory and send each thread's 256 bytes as one asynchronous bulk copy.
// Every mbarrier wait is bounded (status words + CTA-wide abort flag), no TMA multicast is used.
//
// Two forms of the same kernel.  kCtas == 1: every CTA computes its own 128 x 256 tile and has to pull 48 KB per K
// block into shared memory.  kCtas == 2: a cluster of two CTAs computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and HALF of the weight rows (32 KB per K block; the
// tensor core reads the other half from the peer's shared memory), the leader CTA issues the MMAs for both, each CTA
// drains the accumulators of its own rows.  Measured 1.31 against 1.15 PFLOP/s at 32 experts x 1024 rows.  The host
// picks the paired form when the experts are large enough to fill 256-row tiles.
#include <algorithm>
#include <atomic>

#include "tc_ptx.cuh"

namespace epsb {

namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBKBytes = 128;   // bytes of one K block
constexpr int kBKElems = 64;    // bf16 elements of one K block
constexpr int kABytes = kBM * kBKBytes;
constexpr int kThreads = 384;
constexpr int kTmemCols = 512;
constexpr int kMaxExperts = 1024;
constexpr int kOutRowBytes = 256 + 16;
constexpr int kPairRowsPerExpert = 512;   // expected rows per expert from which CTA pairs are used

// tcgen05 instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9 and 10-12 = 1), both
// K-major, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
constexpr uint32_t bf16_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int kCtas>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (kCtas == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// A CTA stages its 128 rows of A and the weight rows it contributes to the MMA: all 256 alone, 128 in a pair.
template <int kCtas>
struct Storage {
  static constexpr int kStages = kCtas == 1 ? 3 : 4;
  static constexpr int kBBytes = (kBN / kCtas) * kBKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  uint8_t tiles[kStages][kStageBytes];
  uint8_t out_stage[2][kBM][kOutRowBytes];
  uint64_t full[kStages];      // in a pair only the leader's are used: both CTAs' copies report to them
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];      // in a pair only the leader's are used: 8 epilogue warps of each CTA arrive
  uint32_t tmem_base;
  volatile int abort_flag;
  int32_t tile_prefix[kMaxExperts + 1];
};

// ---- cluster helpers of the paired form
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a pair: the data lands in this CTA, the bytes are reported to a barrier of either CTA (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// all MMAs this thread issued so far (in both CTAs of the pair) arrive once on the barrier at this cluster address
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

struct Params {
  const int32_t* excl;
  void* C;
  int32_t* status;
  int num_experts;
  int64_t N, K;
  int n_tiles;
};

struct Tile {
  int e, row0, rows_left, n;   // row0 / rows_left: of the whole tile (128 * kCtas rows)
};

template <int kCtas>
__device__ __forceinline__ Tile locate(int t, const Params& p, const Storage<kCtas>* sm) {
  const int g = t / p.n_tiles;
  Tile c;
  c.n = t - g * p.n_tiles;
  int lo = 0, hi = p.num_experts;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sm->tile_prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  c.e = lo;
  const int m = g - sm->tile_prefix[lo];
  const int b = __ldg(p.excl + lo), e_ = __ldg(p.excl + lo + 1);
  c.row0 = b + m * kBM * kCtas;
  c.rows_left = e_ - c.row0;
  return c;
}

template <int kCtas>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const Params p) {
  extern __shared__ uint8_t smem_raw[];
  using St = Storage<kCtas>;
  constexpr int kStages = St::kStages;
  St* sm = reinterpret_cast<St*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (int)(p.K / kBKElems);
  const uint32_t cta = kCtas == 2 ? cluster_ctarank() : 0u;   // 0 = the CTA that issues the MMAs
  const int unit = (int)blockIdx.x / kCtas, units = (int)gridDim.x / kCtas;   // tiles are dealt to CTAs or to pairs

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&sm->tmem_full[b], 1);
      mbar_init(&sm->tmem_empty[b], 8 * kCtas);
    }
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (kCtas == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {   // the same warp of both CTAs, the same destination address
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  if (warp == 2) {
    int carry = 0;
    for (int e0 = 0; e0 < p.num_experts; e0 += 32) {
      const int e = e0 + lane;
      int mt = 0;
      if (e < p.num_experts) mt = (__ldg(p.excl + e + 1) - __ldg(p.excl + e) + kBM * kCtas - 1) / (kBM * kCtas);
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
  if constexpr (kCtas == 2) cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  const int total_tiles = sm->tile_prefix[p.num_experts] * p.n_tiles;

  // 128 * dec + 256 * inc <= 384 * 168: setmaxnreg.inc blocks until the CTA's own register pool can serve it
  static_assert(128 * 40 + 256 * 232 <= kThreads * 168, "setmaxnreg budget exceeds the CTA's register pool");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------ TMA producer (one per CTA).  In a pair each CTA loads its
      // own rows of A and its half of the weight rows; every copy reports its bytes to the LEADER's stage barrier,
      // on which the leader's producer has announced the bytes of both CTAs.
      uint32_t it = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units) {
        const Tile c = locate<kCtas>(t, p, sm);
        const int arow = c.row0 + kBM * (int)cta;
        const int brow = (int)(c.e * p.N + c.n * kBN) + (kBN / kCtas) * (int)cta;
        for (int kb = 0; kb < KB; kb++, it++) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait(&sm->empty[s], ph ^ 1, sm, p.status, 11))) break;
          uint8_t* base = sm->tiles[s];
          if constexpr (kCtas == 1) {
            mbar_expect_tx(&sm->full[s], St::kStageBytes);
            tma_load_2d(base, &tmap_a, kb * kBKElems, arow, &sm->full[s]);
            tma_load_2d(base + kABytes, &tmap_b, kb * kBKElems, brow, &sm->full[s]);
            tma_load_2d(base + 2 * kABytes, &tmap_b, kb * kBKElems, brow + 128, &sm->full[s]);
          } else {
            if (cta == 0) mbar_expect_tx(&sm->full[s], 2 * St::kStageBytes);
            const uint32_t bar = map_to_cta(smem_u32(&sm->full[s]), 0);
            tma_load_2d_pair(base, &tmap_a, kb * kBKElems, arow, bar);
            tma_load_2d_pair(base + kABytes, &tmap_b, kb * kBKElems, brow, bar);
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    } else if (warp == 1 && lane == 0 && cta == 0) {
      // ------------------------------------------------ MMA issuer (the leader's, for both CTAs of a pair)
      constexpr uint32_t idesc = bf16_idesc(kBM * kCtas, kBN);
      uint32_t it = 0, tile_no = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units, tile_no++) {
        const int buf = tile_no & 1;
        const uint32_t tph = (tile_no >> 1) & 1;
        if (!(ok = mbar_wait(&sm->tmem_empty[buf], tph ^ 1, sm, p.status, 21))) break;
        const uint32_t d = tmem_base + (uint32_t)buf * kBN;
        for (int kb = 0; kb < KB; kb++, it++) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait(&sm->full[s], ph, sm, p.status, 22))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sm->tiles[s]);
          const uint64_t da = smem_desc(a_addr), db = smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k4 = 0; k4 < 4; k4++)
            umma_bf16<kCtas>(d, da + 2 * k4, db + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          if constexpr (kCtas == 1) {
            umma_commit(&sm->empty[s]);
          } else {   // the stage is free in both CTAs
            umma_commit_pair(map_to_cta(smem_u32(&sm->empty[s]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&sm->empty[s]), 1));
          }
        }
        if (ok) {
          if constexpr (kCtas == 1) {
            umma_commit(&sm->tmem_full[buf]);
          } else {
            umma_commit_pair(map_to_cta(smem_u32(&sm->tmem_full[buf]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&sm->tmem_full[buf]), 1));
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ------------------------------------------------ epilogue: each CTA drains the accumulators of its own rows
    const int ew = warp - 4, quad = warp & 3, half = ew >> 2;
    const int r_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    uint32_t tile_no = 0;
    bool ok = true;
    for (int t = unit; t < total_tiles && ok; t += units, tile_no++) {
      const Tile c = locate<kCtas>(t, p, sm);
      const int buf = tile_no & 1;
      ok = mbar_wait(&sm->tmem_full[buf], (tile_no >> 1) & 1u, sm, p.status, 31);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row_in_unit = kBM * (int)cta + r_in_tile;
      const int64_t grow = (int64_t)c.row0 + row_in_unit;
      const int64_t col0 = (int64_t)c.n * kBN + 128 * half;
      const bool store = row_in_unit < c.rows_left && col0 < p.N;
      uint8_t* stage_row = sm->out_stage[half][r_in_tile];
      bulk_wait_read();  // this thread's copy of the previous tile has left the staging row
      const uint32_t tb = lane_addr + (uint32_t)buf * kBN + (uint32_t)(128 * half);
      uint32_t v0[32], v1[32];
#pragma unroll
      for (int ch = 0; ch < 4; ch += 2) {
        tmem_ld32_async(tb + ch * 32, v0);
        tmem_ld32_async(tb + ch * 32 + 32, v1);
        tmem_wait(v0);
        tmem_tie(v1);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v0[q * 8 + 0]), __uint_as_float(v0[q * 8 + 1]));
          o.y = pack_bf16x2(__uint_as_float(v0[q * 8 + 2]), __uint_as_float(v0[q * 8 + 3]));
          o.z = pack_bf16x2(__uint_as_float(v0[q * 8 + 4]), __uint_as_float(v0[q * 8 + 5]));
          o.w = pack_bf16x2(__uint_as_float(v0[q * 8 + 6]), __uint_as_float(v0[q * 8 + 7]));
          st_shared_16(stage_row + ch * 64 + q * 16, o);
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v1[q * 8 + 0]), __uint_as_float(v1[q * 8 + 1]));
          o.y = pack_bf16x2(__uint_as_float(v1[q * 8 + 2]), __uint_as_float(v1[q * 8 + 3]));
          o.z = pack_bf16x2(__uint_as_float(v1[q * 8 + 4]), __uint_as_float(v1[q * 8 + 5]));
          o.w = pack_bf16x2(__uint_as_float(v1[q * 8 + 6]), __uint_as_float(v1[q * 8 + 7]));
          st_shared_16(stage_row + (ch + 1) * 64 + q * 16, o);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtas == 1) mbar_arrive(&sm->tmem_empty[buf]);
        else mbar_arrive_cluster(map_to_cta(smem_u32(&sm->tmem_empty[buf]), 0));
      }
      if (store) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        bulk_store_row(reinterpret_cast<uint8_t*>(p.C) + (grow * p.N + col0) * 2, stage_row, 256);
        bulk_commit();
      }
    }
    bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  // a pair leaves together: the leader's MMAs read the peer's shared memory and the peer arrives on the leader's barriers
  if constexpr (kCtas == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (kCtas == 1)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

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

// 2-D bf16 tensor [rows, K] (K contiguous), box 64 elements (128 bytes) x 128 rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return fail(EPSB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBKElems, 128u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EPSB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return EPSB_OK;
}

}  // namespace

}  // namespace epsb

using namespace epsb;

namespace {

template <int kCtas>
int launch_bf16(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int64_t tiles_max, int sm_count,
                cudaStream_t st) {
  const size_t smem = sizeof(Storage<kCtas>) + 1024;
  static std::atomic<int> max_units[64];   // per device: 0 = not configured yet, else CTAs (or pairs) that fit at once
  int dev = 0;
  cudaGetDevice(&dev);
  int fit = (dev >= 0 && dev < 64) ? max_units[dev].load(std::memory_order_acquire) : 0;
  if (fit == 0) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_bf16_kernel<kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaFuncSetAttribute(gemm bf16): %s", cudaGetErrorString(e));
    fit = gemm_cta_limit(0);
    if (kCtas == 2) {
      // how many PAIRS the device can hold at once (a pair needs two SMs of one cluster-capable group)
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * gemm_cta_limit(0));
      q.blockDim = dim3(kThreads);
      q.dynamicSmemBytes = smem;
      cudaLaunchAttribute a[1];
      a[0].id = cudaLaunchAttributeClusterDimension;
      a[0].val.clusterDim.x = 2;
      a[0].val.clusterDim.y = 1;
      a[0].val.clusterDim.z = 1;
      q.attrs = a;
      q.numAttrs = 1;
      int clusters = 0;
      e = cudaOccupancyMaxActiveClusters(&clusters, grouped_gemm_bf16_kernel<kCtas>, &q);
      if (e != cudaSuccess || clusters <= 0)
        return fail(EPSB_ERR_CUDA, "cudaOccupancyMaxActiveClusters(gemm bf16 pairs): %s", cudaGetErrorString(e));
      fit = clusters;
    }
    if (dev >= 0 && dev < 64) max_units[dev].store(fit, std::memory_order_release);
  }
  int64_t units = tiles_max;
  int64_t limit = kCtas == 1 ? gemm_cta_limit(sm_count) : std::min<int64_t>(fit, gemm_cta_limit(sm_count) / 2);
  if (limit < 1) limit = 1;
  if (units > limit) units = limit;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(units * kCtas));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, grouped_gemm_bf16_kernel<kCtas>, ta, tb, p);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "grouped_gemm_bf16 launch: %s", cudaGetErrorString(e));
  return check_launch("grouped_gemm_bf16");
}

}  // namespace

extern "C" int epsb_grouped_gemm_bf16(const void* A, const void* B, const int32_t* excl, int num_experts,
                                      int64_t max_rows, int64_t rows_hint, int64_t N, int64_t K, void* C,
                                      int32_t* status, int sm_count, void* stream) {
  EPSB_REQUIRE(sm_count >= 0, EPSB_ERR_INVALID, "sm_count %d is negative", sm_count);
  EPSB_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts, EPSB_ERR_INVALID, "num_experts %d out of range",
               num_experts);
  EPSB_REQUIRE(K > 0 && K % 64 == 0, EPSB_ERR_INVALID, "K: %lld is not divisible by 64", (long long)K);
  EPSB_REQUIRE(N > 0 && N % 128 == 0, EPSB_ERR_INVALID, "N: %lld is not divisible by 128", (long long)N);
  EPSB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0, EPSB_ERR_INVALID,
               "A, B and C must be 16-byte aligned");
  EPSB_REQUIRE((int64_t)num_experts * N < (1ll << 31) && max_rows < (1ll << 31), EPSB_ERR_INVALID,
               "tensor too large for 32-bit TMA coordinates");
  EPSB_REQUIRE(rows_hint >= 0, EPSB_ERR_INVALID, "rows_hint %lld is negative", (long long)rows_hint);
  if (max_rows <= 0) return EPSB_OK;
  CUtensorMap ta, tb;
  int rc = make_map(&ta, A, max_rows, K);
  if (rc) return rc;
  rc = make_map(&tb, B, (int64_t)num_experts * N, K);
  if (rc) return rc;
  Params p;
  p.excl = excl;
  p.C = C;
  p.status = status;
  p.num_experts = num_experts;
  p.N = N;
  p.K = K;
  p.n_tiles = (int)((N + kBN - 1) / kBN);
  // Pairs pay when the experts fill 256-row tiles (measured: +14 % at 512 and 1024 rows per expert, -6 % at
  // 300 +- 40 rows, where every expert's last pair tile is half empty); the row counts live on the device, so the
  // choice goes by the caller's expectation (the reference's num_tokens_hint), else by the capacity.  N must split
  // into two 128-row halves per tile for a pair.
  const int64_t expected = rows_hint > 0 ? std::min(rows_hint, max_rows) : max_rows;
  const bool pairs = N % kBN == 0 && expected >= (int64_t)num_experts * kPairRowsPerExpert && sm_count != 1;
  auto st = static_cast<cudaStream_t>(stream);
  if (pairs) {
    const int64_t tiles_max = ((max_rows + 2 * kBM - 1) / (2 * kBM) + num_experts) * p.n_tiles;
    return launch_bf16<2>(ta, tb, p, tiles_max, sm_count, st);
  }
  const int64_t tiles_max = ((max_rows + kBM - 1) / kBM + num_experts) * p.n_tiles;
  return launch_bf16<1>(ta, tb, p, tiles_max, sm_count, st);
}
