// FP8 block-scaled grouped GEMM, "token-N" orientation (sm_100a).
//
// Same arithmetic as grouped_gemm.cu, with the operand roles swapped (what the reference does on H20 with its
// swap-AB tiles, src/gemm/aok_grouped_gemm/src/operations/hopper_grouped_gemm.cu:147-170): the 128 rows of a WEIGHT
// tile are the MMA's M (TMEM lanes) and an expert's tokens are its N (TMEM columns, any multiple of 16 up to 256).
// An expert of up to tile_tokens rows is then ONE tile whatever its row count and streams its weights exactly once;
// the accumulator is tile_tokens columns wide, so 512 / round32(tile_tokens) K steps fit in TMEM at once.
//
// Roles (384 threads, one CTA per SM, persistent over a device-built tile list):
//   warp 0    TMA producer: weight tile (128 x 128 B) + token rows (boxes of 256/128/64/32/16 rows) per K step
//   warp 1    MMA issuer (tcgen05.mma kind::f8f6f4, M128, N = tokens of the tile), TMEM allocation
//   warps 2,3 scale loaders: a_s[token, kb] * b_s[block, kb] for the tile's tokens into a shared-memory ring, in
//             batches of four K steps (the epilogue needs one scale per COLUMN in this orientation)
//   warps 4-11 epilogue: drain TMEM per K step with the 16x256b load shape, fold into fp32 registers, then
//             transpose the tile through warp-private shared memory and store coalesced 16-byte pieces
// Every mbarrier wait is bounded (status words as in grouped_gemm.cu); no TMA multicast.
//
// Where it stands: the per-K-step synchronisation chain of the epilogue (two waits, TMEM loads, release) costs
// about as much for 128 weight rows here as for 256 in grouped_gemm.cu, so at 128 rows per expert this kernel
// runs at about 60 % of the other one's speed and the host side does not select it by default; it is kept as the
// drop-in for callers that want the reference's swapped orientation and as the base for a leaner K loop.
#include "tc_ptx.cuh"


namespace epsb {

namespace {

constexpr int kThreads = 384;
constexpr int kWRows = 128;             // weight rows per tile = MMA M
constexpr int kBK = 128;
constexpr int kWBytes = kWRows * kBK;   // 16 KB
constexpr int kMaxStages = 8;
constexpr int kMaxBuf = 8;
constexpr int kScaleBatches = 3;  // batches of four K steps in the scale ring
constexpr int kMaxExperts = 1024;
constexpr int kOutRowBytes = 64 + 16;   // one warp's 32 weight rows of one token (bf16) + padding
constexpr int kSmemLimit = 232448;      // 227 KB

struct TnParams {
  const float* a_s;
  const float* b_s;
  const int32_t* excl;
  void* C;
  const float* row_w;
  int32_t* status;
  int num_experts;
  int64_t max_rows;
  int64_t N;          // weight rows per expert
  int64_t K;
  int w_tiles;        // N / 128
  int tile_tokens;    // tokens per tile (multiple of 16, <= 256)
  int col_stride;     // TMEM columns per accumulator buffer (multiple of 32)
  int n_buf;          // accumulator buffers in TMEM
  int n_stages;       // TMA ring depth
  int stage_bytes;    // 16 KB + tile_tokens * 128, multiple of 1024
  int ctrl_off, scale_off, out_off;  // byte offsets of the regions behind the tile ring
  int half_rows;      // token columns one epilogue warp can hold in its output staging area
};

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kMaxBuf];
  uint64_t tmem_empty[kMaxBuf];
  uint64_t sc_full[kScaleBatches];   // one phase per batch of four K steps
  uint64_t sc_empty[kScaleBatches];
  uint32_t tmem_base;
  volatile int abort_flag;
  alignas(16) float row_w[8][128];    // per epilogue warp: the gate weights of its token columns (down mode)
  int32_t tile_prefix[kMaxExperts + 1];  // token tiles before each expert
};

struct Tile {
  int e, w, row0, valid, ncols;  // expert, weight tile, first GEMM row, valid tokens, columns (valid rounded to 16)
};

__device__ __forceinline__ Tile locate(int t, const TnParams& p, const Ctrl* c) {
  const int g = t / p.w_tiles;
  Tile tl;
  tl.w = t - g * p.w_tiles;
  int lo = 0, hi = p.num_experts;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (c->tile_prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  tl.e = lo;
  const int m = g - c->tile_prefix[lo];
  const int b = __ldg(p.excl + lo), e_ = __ldg(p.excl + lo + 1);
  tl.row0 = b + m * p.tile_tokens;
  tl.valid = min(p.tile_tokens, e_ - tl.row0);
  tl.ncols = (tl.valid + 15) & ~15;
  return tl;
}

struct TokenMaps {
  CUtensorMap box[5];  // boxes of 256, 128, 64, 32, 16 token rows x 128 bytes
};

template <int kMode, int kCh>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_fp8_tn_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ TokenMaps tmap_a,
                           const TnParams p) {
  extern __shared__ uint8_t smem_raw_tn[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_tn) + 1023) & ~(uintptr_t)1023);
  Ctrl* sm = reinterpret_cast<Ctrl*>(base + p.ctrl_off);
  float* sc_ring = reinterpret_cast<float*>(base + p.scale_off);        // [kScaleBatches][4][col_stride]
  uint8_t* out_stage = base + p.out_off;                                // [8 warps][half_rows tokens][kOutRowBytes]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (int)(p.K / kBK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; s++) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], 1);
    }
    for (int b = 0; b < kMaxBuf; b++) {
      mbar_init(&sm->tmem_full[b], 1);
      mbar_init(&sm->tmem_empty[b], 8);   // one arrival per epilogue warp
    }
    for (int s = 0; s < kScaleBatches; s++) {
      mbar_init(&sm->sc_full[s], 2);      // one arrival per loader warp
      mbar_init(&sm->sc_empty[s], 8);     // one arrival per epilogue warp
    }
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp == 2) {
    int carry = 0;
    for (int e0 = 0; e0 < p.num_experts; e0 += 32) {
      const int e = e0 + lane;
      int mt = 0;
      if (e < p.num_experts) mt = (__ldg(p.excl + e + 1) - __ldg(p.excl + e) + p.tile_tokens - 1) / p.tile_tokens;
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
  const int total_tiles = sm->tile_prefix[p.num_experts] * p.w_tiles;

  // register budget: see grouped_gemm.cu (128 * dec + 256 * inc <= 384 * 168)
  static_assert(128 * 72 + 256 * 208 <= kThreads * 168, "setmaxnreg budget exceeds the CTA's register pool");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------ TMA producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tl = locate(t, p, sm);
        const int wrow = (int)(tl.e * p.N + (int64_t)tl.w * kWRows);
        for (int kb = 0; kb < KB; kb++) {
          if (!(ok = mbar_wait(&sm->empty[s], ph ^ 1, sm, p.status, 11))) break;
          mbar_expect_tx(&sm->full[s], kWBytes + tl.ncols * kBK);
          uint8_t* st = base + (size_t)s * p.stage_bytes;
          tma_load_2d(st, &tmap_w, kb * kBK, wrow, &sm->full[s]);
          // token rows: greedy split of ncols (a multiple of 16) into boxes of 256/128/64/32/16 rows
          int done = 0;
#pragma unroll
          for (int b = 0; b < 5; b++) {
            const int rows = 256 >> b;
            if (tl.ncols - done >= rows) {
              tma_load_2d(st + kWBytes + done * kBK, &tmap_a.box[b], kb * kBK, tl.row0 + done, &sm->full[s]);
              done += rows;
            }
          }
          if (++s == p.n_stages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------ MMA issuer
      int s = 0, buf = 0;
      uint32_t ph = 0, tph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tl = locate(t, p, sm);
        const uint32_t idesc = f8_idesc(kWRows, tl.ncols);
        for (int kb = 0; kb < KB; kb++) {
          if (!(ok = mbar_wait(&sm->tmem_empty[buf], tph ^ 1, sm, p.status, 21))) break;
          if (!(ok = mbar_wait(&sm->full[s], ph, sm, p.status, 22))) break;
          tc_fence_after();
          const uint32_t w_addr = smem_u32(base + (size_t)s * p.stage_bytes);
          const uint64_t da = smem_desc(w_addr);            // A operand: the weight tile
          const uint64_t db = smem_desc(w_addr + kWBytes);  // B operand: the token rows
          const uint32_t d = tmem_base + (uint32_t)(buf * p.col_stride);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; k4++) umma_f8(d, da + 2 * k4, db + 2 * k4, idesc, k4 > 0 ? 1u : 0u);
          umma_commit(&sm->empty[s]);
          umma_commit(&sm->tmem_full[buf]);
          if (++s == p.n_stages) {
            s = 0;
            ph ^= 1;
          }
          if (++buf == p.n_buf) {
            buf = 0;
            tph ^= 1;
          }
        }
      }
    } else if (warp >= 2) {
      // ------------------------------------------------ scale loaders (64 threads)
      // Batches of four K steps, four token columns per thread; the loads of batch i+1 are in flight while
      // batch i is written to the ring.
      const int lt = (warp - 2) * 32 + lane;
      const int NBw = (int)(p.N / 128);
      const bool vec = (KB & 3) == 0;
      struct Batch {
        int t, kb0;
        Tile tl;
        bool live;
      };
      auto fetch = [&](const Batch& b, float4 (&v)[4], float4& sb) {
        const float* bs = p.b_s + ((int64_t)b.tl.e * NBw + b.tl.w) * KB + b.kb0;
        const int nk = min(4, KB - b.kb0);
        if (vec) {
          sb = __ldg(reinterpret_cast<const float4*>(bs));
        } else {
          sb.x = __ldg(bs);
          sb.y = nk > 1 ? __ldg(bs + 1) : 0.0f;
          sb.z = nk > 2 ? __ldg(bs + 2) : 0.0f;
          sb.w = nk > 3 ? __ldg(bs + 3) : 0.0f;
        }
#pragma unroll
        for (int ci = 0; ci < 4; ci++) {
          const int c = lt + ci * 64;
          const int64_t row = (int64_t)b.tl.row0 + c;
          v[ci] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (c < b.tl.valid && row < p.max_rows) {
            const float* as = p.a_s + row * KB + b.kb0;
            if (vec) {
              v[ci] = __ldg(reinterpret_cast<const float4*>(as));
            } else {
              v[ci].x = __ldg(as);
              if (nk > 1) v[ci].y = __ldg(as + 1);
              if (nk > 2) v[ci].z = __ldg(as + 2);
              if (nk > 3) v[ci].w = __ldg(as + 3);
            }
          }
        }
      };
      auto advance = [&](Batch& b) {
        b.kb0 += 4;
        if (b.kb0 >= KB) {
          b.kb0 = 0;
          b.t += gridDim.x;
          b.live = b.t < total_tiles;
          if (b.live) b.tl = locate(b.t, p, sm);
        }
      };
      Batch cur;
      cur.t = blockIdx.x;
      cur.kb0 = 0;
      cur.live = cur.t < total_tiles;
      float4 v[4], sb;
      if (cur.live) {
        cur.tl = locate(cur.t, p, sm);
        fetch(cur, v, sb);
      }
      int slot = 0;
      uint32_t sph = 0;
      bool ok = true;
      while (cur.live && ok) {
        Batch nxt = cur;
        advance(nxt);
        float4 nv[4], nsb;
        if (nxt.live) fetch(nxt, nv, nsb);
        const int nk = min(4, KB - cur.kb0);
        ok = mbar_wait(&sm->sc_empty[slot], sph ^ 1, sm, p.status, 51);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        float* dst = sc_ring + slot * 4 * p.col_stride;
#pragma unroll
        for (int ci = 0; ci < 4; ci++) {
          const int c = lt + ci * 64;
          if (c < cur.tl.ncols) {
            dst[c] = v[ci].x * sb.x;
            if (nk > 1) dst[p.col_stride + c] = v[ci].y * sb.y;
            if (nk > 2) dst[2 * p.col_stride + c] = v[ci].z * sb.z;
            if (nk > 3) dst[3 * p.col_stride + c] = v[ci].w * sb.w;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->sc_full[slot]);
        if (++slot == kScaleBatches) {
          slot = 0;
          sph ^= 1;
        }
        cur = nxt;
#pragma unroll
        for (int ci = 0; ci < 4; ci++) v[ci] = nv[ci];
        sb = nsb;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // ------------------------------------------------ epilogue: 8 warps
    // Warp w drains TMEM lanes 32*(w%4).. (weight rows) of one half of the tile's token columns, with the
    // 16x256b load shape: thread t holds rows t/4 + {0, 8, 16, 24} of its quadrant and, per 16-column chunk,
    // columns 2*(t%4) + {0, 1, 8, 9}.  A thread therefore needs only 4 scales per chunk and K step (two 8-byte
    // shared-memory loads, conflict-free), where a row-per-thread layout needs all 16 (broadcast loads that
    // saturate the shared-memory pipe).  A tcgen05.ld costs a few hundred cycles from issue to the first use
    // of its registers whatever its width, so all loads of a K step (kBatch chunks) are issued before one wait.
    constexpr int kBatch = kCh <= 4 ? kCh : (kCh == 5 ? 3 : 2);
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;    // which half of the tile's token columns
    const int tq = lane & 3, tr = lane >> 2;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int ew = warp - 4;             // epilogue warp 0..7
    uint8_t* my_stage = out_stage + (size_t)ew * p.half_rows * kOutRowBytes;   // private to this warp
    float* my_w = sm->row_w[ew];
    uint32_t tph = 0, sph = 0;
    int buf = 0, slot = 0;
    bool ok = true;
    auto release_tmem = [&](int b) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->tmem_empty[b]);
    };
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tl = locate(t, p, sm);
      const int nch = tl.ncols >> 4;                  // 16-column chunks in the tile
      const int ch0 = half == 0 ? 0 : (nch + 1) >> 1; // first chunk of this half
      const int my_n = half == 0 ? (nch + 1) >> 1 : nch >> 1;
      float acc[kCh * 16];   // [chunk][lane half 0/1][register of the 16x256b.x2 fragment]
#pragma unroll
      for (int i = 0; i < kCh * 16; i++) acc[i] = 0.0f;

      for (int kb = 0; kb < KB; kb++) {
        ok = mbar_wait(&sm->tmem_full[buf], tph, sm, p.status, 31);
        if (ok && (kb & 3) == 0) ok = mbar_wait(&sm->sc_full[slot], sph, sm, p.status, 32);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tb = lane_addr + (uint32_t)(buf * p.col_stride) + (uint32_t)(ch0 * 16);
        const float* sc = sc_ring + (slot * 4 + (kb & 3)) * p.col_stride + ch0 * 16 + 2 * tq;
#pragma unroll
        for (int b0 = 0; b0 < kCh; b0 += kBatch) {
          if (b0 < my_n) {  // warp-uniform
            uint32_t v[kBatch][2][8];
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
              if (b0 + j < my_n) {
                tmem_ld_frag16_async(tb + (uint32_t)((b0 + j) * 16), v[j][0]);
                tmem_ld_frag16_async(tb + (16u << 16) + (uint32_t)((b0 + j) * 16), v[j][1]);
              }
            }
            tmem_wait8(v[0][0]);
            tmem_tie8(v[0][1]);
#pragma unroll
            for (int j = 1; j < kBatch; j++) {
              if (b0 + j < my_n) {
                tmem_tie8(v[j][0]);
                tmem_tie8(v[j][1]);
              }
            }
            if (b0 + kBatch >= my_n) release_tmem(buf);  // this K step's last loads have landed
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
              if (b0 + j < my_n) {
                const float2 lo = *reinterpret_cast<const float2*>(sc + (b0 + j) * 16);
                const float2 hi = *reinterpret_cast<const float2*>(sc + (b0 + j) * 16 + 8);
#pragma unroll
                for (int hs = 0; hs < 2; hs++) {
                  float* a = &acc[(b0 + j) * 16 + hs * 8];
                  const uint32_t* r = v[j][hs];
                  a[0] = fmaf(__uint_as_float(r[0]), lo.x, a[0]);
                  a[1] = fmaf(__uint_as_float(r[1]), lo.y, a[1]);
                  a[2] = fmaf(__uint_as_float(r[2]), lo.x, a[2]);
                  a[3] = fmaf(__uint_as_float(r[3]), lo.y, a[3]);
                  a[4] = fmaf(__uint_as_float(r[4]), hi.x, a[4]);
                  a[5] = fmaf(__uint_as_float(r[5]), hi.y, a[5]);
                  a[6] = fmaf(__uint_as_float(r[6]), hi.x, a[6]);
                  a[7] = fmaf(__uint_as_float(r[7]), hi.y, a[7]);
                }
              }
            }
          }
        }
        if (my_n == 0) release_tmem(buf);  // a half without columns (16-token tiles) still owes its arrival
        if (++buf == p.n_buf) {
          buf = 0;
          tph ^= 1;
        }
        if ((kb & 3) == 3 || kb == KB - 1) {  // last K step of a scale batch: hand the batch back
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm->sc_empty[slot]);
          if (++slot == kScaleBatches) {
            slot = 0;
            sph ^= 1;
          }
        }
      }
      if (!ok) break;

      // ---- tile epilogue, warp-private (no barrier between warps): the warp's 32 weight rows x its token
      // columns are transposed through its own staging rows (one per token column, 64 bytes of bf16) and leave
      // as coalesced 16-byte stores.  (Bulk copies are too slow here: the copy engine takes one small copy every
      // few cycles, and a tile has hundreds of 64-byte pieces.)
      const int col_base = ch0 * 16;               // first token column of this half
      const int my_cols = min(my_n * 16, tl.valid - col_base);   // token columns this warp stores (may be <= 0)
      __syncwarp();                                // every lane has read the previous tile's staging rows
      if (kMode == EPSB_GEMM_DOWN && p.row_w != nullptr) {
        for (int c = lane; c < my_n * 16; c += 32)
          my_w[c] = c < my_cols ? __ldg(p.row_w + tl.row0 + col_base + c) : 0.0f;
        __syncwarp();
      }
      // Lanes t and t^4 hold adjacent weight rows of the same columns: they swap one value per column pair, so
      // that each lane stores packed bf16x2 words (two weight rows of one token column); a warp's 32 words of
      // one store fall into 32 distinct banks (row pitch 80 bytes).
      {
        const int odd = tr & 1;
#pragma unroll
        for (int ch = 0; ch < kCh; ch++) {
          if (ch < my_n) {
            float2 wlo = make_float2(1.0f, 1.0f), whi = wlo;
            if (kMode == EPSB_GEMM_DOWN && p.row_w != nullptr) {
              wlo = *reinterpret_cast<const float2*>(my_w + ch * 16 + 2 * tq);
              whi = *reinterpret_cast<const float2*>(my_w + ch * 16 + 2 * tq + 8);
            }
#pragma unroll
            for (int hs = 0; hs < 2; hs++) {
#pragma unroll
              for (int r = 0; r < 8; r += 2) {
                const float wx = (r & 4) ? whi.x : wlo.x, wy = (r & 4) ? whi.y : wlo.y;
                const float a = acc[ch * 16 + hs * 8 + r] * wx, b = acc[ch * 16 + hs * 8 + r + 1] * wy;
                const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 4);
                const uint32_t word = odd ? pack_bf16x2(got, b) : pack_bf16x2(a, got);
                const int col = ch * 16 + 2 * tq + ((r & 4) ? 8 : 0) + odd;
                const int lrow = hs * 16 + (tr & ~1) + ((r & 2) ? 8 : 0);   // weight row inside the quadrant
                *reinterpret_cast<uint32_t*>(my_stage + (size_t)col * kOutRowBytes + lrow * 2) = word;
              }
            }
          }
        }
      }
      __syncwarp();
      // 16-byte pieces back out of the staging rows: four lanes cover one token's 64 bytes, so a warp-wide store
      // writes eight whole 64-byte segments of C.
      {
        uint8_t* c_base = reinterpret_cast<uint8_t*>(p.C) +
                          (((int64_t)tl.row0 + col_base) * p.N + (int64_t)tl.w * kWRows + quad * 32) * 2 + tq * 16;
#pragma unroll
        for (int i = 0; i < kCh * 2; i++) {
          const int c = i * 8 + tr;
          if (c < my_cols) {
            const uint4 v = *reinterpret_cast<const uint4*>(my_stage + (size_t)c * kOutRowBytes + tq * 16);
            st_16(c_base + (int64_t)c * p.N * 2, v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn_tn() {
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

// 2-D e4m3 tensor [rows, K] (K contiguous), box `box_rows` x 128 bytes, 128-byte swizzle.
int make_map_tn(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows) {
  EncodeFn fn = encode_fn_tn();
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

}  // namespace

namespace {
int launch_grouped_gemm_tn(int mode, const void* A, const float* a_s, const void* B, const float* b_s,
                           const int32_t* excl, int num_experts, int64_t max_rows, int64_t N, int64_t K, void* C,
                           const float* row_w, int32_t* status, int tile_tokens, int sm_count, cudaStream_t stream) {
  EPSB_REQUIRE(tile_tokens >= 16 && tile_tokens <= 256 && tile_tokens % 16 == 0, EPSB_ERR_INVALID,
               "tile_tokens %d must be a multiple of 16 in [16, 256]", tile_tokens);
  TnParams p;
  p.a_s = a_s; p.b_s = b_s; p.excl = excl; p.C = C; p.row_w = row_w; p.status = status;
  p.num_experts = num_experts; p.max_rows = max_rows; p.N = N; p.K = K;
  p.w_tiles = (int)(N / kWRows);
  p.tile_tokens = tile_tokens;
  p.col_stride = (tile_tokens + 31) & ~31;
  p.n_buf = 512 / p.col_stride;
  if (p.n_buf > kMaxBuf) p.n_buf = kMaxBuf;
  p.stage_bytes = kWBytes + ((tile_tokens * kBK + 1023) & ~1023);
  const int ctrl_bytes = (int)((sizeof(Ctrl) + 127) & ~(size_t)127);
  const int scale_bytes = kScaleBatches * 4 * p.col_stride * 4;
  p.half_rows = ((tile_tokens / 16 + 1) / 2) * 16;
  const int out_bytes = 8 * p.half_rows * kOutRowBytes;
  const int fixed = ctrl_bytes + scale_bytes + out_bytes + 1024 + 128;
  p.n_stages = (kSmemLimit - fixed) / p.stage_bytes;
  if (p.n_stages > kMaxStages) p.n_stages = kMaxStages;
  EPSB_REQUIRE(p.n_stages >= 2, EPSB_ERR_INVALID, "not enough shared memory for two pipeline stages");
  p.ctrl_off = p.n_stages * p.stage_bytes;
  p.scale_off = p.ctrl_off + ctrl_bytes;
  p.out_off = p.scale_off + ((scale_bytes + 127) & ~127);
  const size_t smem = (size_t)p.out_off + out_bytes + 1024;
  EPSB_REQUIRE(smem <= (size_t)kSmemLimit, EPSB_ERR_INVALID, "shared-memory plan of %zu bytes exceeds the limit", smem);

  CUtensorMap tw;
  TokenMaps ta;
  int rc = make_map_tn(&tw, B, (int64_t)num_experts * N, K, kWRows);
  if (rc) return rc;
  for (int b = 0; b < 5; b++) {
    rc = make_map_tn(&ta.box[b], A, max_rows, K, 256 >> b);
    if (rc) return rc;
  }
  const int64_t tok_tiles_max = (max_rows + tile_tokens - 1) / tile_tokens + num_experts;
  int64_t grid = tok_tiles_max * p.w_tiles;
  if (grid > gemm_cta_limit(sm_count)) grid = gemm_cta_limit(sm_count);
  // kCh: 16-column chunks one column half can hold (sets the epilogue's register arrays)
  const int chunks_per_half = (tile_tokens / 16 + 1) / 2;
  const auto st = stream;
#define EPSB_TN_LAUNCH(MODE, CH)                                                                                  \
  do {                                                                                                            \
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_fp8_tn_kernel<MODE, CH>,                                    \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);                \
    if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaFuncSetAttribute(gemm tn): %s", cudaGetErrorString(e)); \
    grouped_gemm_fp8_tn_kernel<MODE, CH><<<(int)grid, kThreads, smem, st>>>(tw, ta, p);                           \
  } while (0)
#define EPSB_TN_MODE(MODE)                                   \
  do {                                                       \
    if (chunks_per_half <= 4) EPSB_TN_LAUNCH(MODE, 4);       \
    else if (chunks_per_half <= 5) EPSB_TN_LAUNCH(MODE, 5);  \
    else EPSB_TN_LAUNCH(MODE, 8);                            \
  } while (0)
  if (mode == EPSB_GEMM_DOWN) EPSB_TN_MODE(EPSB_GEMM_DOWN);
  else EPSB_TN_MODE(EPSB_GEMM_PLAIN);
#undef EPSB_TN_MODE
#undef EPSB_TN_LAUNCH
  return check_launch("grouped_gemm_fp8_tn");
}
}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_grouped_gemm_fp8_tn(int mode, const void* A, const float* a_s, const void* B, const float* b_s,
                                        const int32_t* excl, int num_experts, int64_t max_rows, int64_t N, int64_t K,
                                        void* C, const float* row_w, int32_t* status, int tile_tokens, int sm_count,
                                        void* stream) {
  EPSB_REQUIRE(sm_count >= 0, EPSB_ERR_INVALID, "sm_count %d is negative", sm_count);
  EPSB_REQUIRE(mode == EPSB_GEMM_PLAIN || mode == EPSB_GEMM_DOWN, EPSB_ERR_INVALID,
               "token-N GEMM supports modes PLAIN and DOWN, got %d", mode);
  EPSB_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts, EPSB_ERR_INVALID, "num_experts %d out of range",
               num_experts);
  EPSB_REQUIRE(K > 0 && K % 128 == 0, EPSB_ERR_INVALID, "K: %lld is not divisible by 128", (long long)K);
  EPSB_REQUIRE(N > 0 && N % 128 == 0, EPSB_ERR_INVALID, "N: %lld is not divisible by 128", (long long)N);
  EPSB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)B & 15) == 0 && ((uintptr_t)C & 15) == 0 &&
                   ((uintptr_t)a_s & 15) == 0 && ((uintptr_t)b_s & 15) == 0,
               EPSB_ERR_INVALID, "A, B, C and the scale arrays must be 16-byte aligned");
  EPSB_REQUIRE((int64_t)num_experts * N < (1ll << 31) && max_rows < (1ll << 31), EPSB_ERR_INVALID,
               "tensor too large for 32-bit TMA coordinates");
  if (max_rows <= 0) return EPSB_OK;
  return launch_grouped_gemm_tn(mode, A, a_s, B, b_s, excl, num_experts, max_rows, N, K, C, row_w, status, tile_tokens,
                                sm_count, static_cast<cudaStream_t>(stream));
}
