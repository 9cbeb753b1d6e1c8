/*
 * CPU restatement of the eps FP8 MoE expert-layer path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the
 * tests, the smoke check and the benchmark's cpu_baseline / reference arm load
 * it.  Nothing in the product package may link, import or call it.
 *
 * Every function names the reference file:line it restates.  The plan functions
 * simulate the reference kernels' thread decomposition literally (an outer loop
 * over the thread id) because the row orders the reference produces are
 * artefacts of that decomposition.
 *
 * Parity pin: the reference ships no tests, golden vectors or fixtures for this
 * path.  The pin is the reference's own arch-agnostic kernels compiled from its
 * sources (oracle/ref_harness.cu -> oracle/_ref/) and run on a B200; fixtures
 * recorded from that run live in tests/golden/ and tests/test_oracle_golden.py
 * checks this file against them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CEILDIV(a, b) (((a) + (b)-1) / (b))

/* ------------------------------------------------------------------ scalar formats */

static inline float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_as_u32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float orc_bf16_to_f32(uint16_t h) { return u32_as_f32((uint32_t)h << 16); }

/* float -> bf16, round to nearest even (what __float2bfloat16_rn does). */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f32_as_u32(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* float -> FP8 e4m3 (fn variant: no inf, max 448), round to nearest even,
 * saturate to +-448; what cvt.rn.satfinite.e4m3x2.f32 does (cuda_fp8.hpp,
 * used by quant/fp8.cu:288). */
uint8_t orc_f32_to_e4m3(float f) {
  uint32_t bits = f32_as_u32(f);
  uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
  uint32_t u = bits & 0x7fffffffu;
  if (u > 0x7f800000u) return (uint8_t)(sign | 0x7f);  /* NaN */
  if (u >= 0x43e00000u) return (uint8_t)(sign | 0x7e); /* >= 448 saturates */
  if (u < 0x3c800000u) {                               /* below 2^-6: subnormal grid of 2^-9 */
    float a = u32_as_f32(u);
    int q = (int)nearbyintf(a * 512.0f);               /* exact product; ties to even */
    return (uint8_t)(sign | (uint8_t)q);
  }
  uint32_t lsb = (u >> 20) & 1u;
  u += 0x7ffffu + lsb;
  u >>= 20;
  uint32_t code = u - ((127u - 7u) << 3);
  if (code > 0x7e) code = 0x7e;
  return (uint8_t)(sign | (uint8_t)code);
}

float orc_e4m3_to_f32(uint8_t c) {
  int sign = c & 0x80;
  int e = (c >> 3) & 0xf;
  int m = c & 7;
  float v;
  if (e == 0xf && m == 7) return NAN;
  if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return sign ? -v : v;
}

void orc_e4m3_table(float* out256) {
  for (int i = 0; i < 256; i++) out256[i] = orc_e4m3_to_f32((uint8_t)i);
}

/* ------------------------------------------------------------------ Q1 / Q2 quant */

/*
 * Per-row, per-128-column FP8 quantisation.  quant/fp8.cu:247-296:
 *   amax over the group (starting from 0.0f, fabs of the fp32 value),
 *   scale = amax / 448, written to scales[row, group] (row-major),
 *   inv   = 1 / scale,
 *   code  = e4m3_rn_satfinite(fmax(-448, fmin(x * inv, 448))).
 * An all-zero group gives scale 0, inv +inf, 0*inf = NaN, and fmin/fmax drop
 * the NaN operand, so every code of that group is 0x7E (+448) and dequantises to
 * 448*0 = 0.  C fminf/fmaxf have the same NaN rule as the CUDA ones.
 *
 * div_mode 1 (default of the product, what the reference kernel computes):
 *   scale = div.full.f32(amax, 448) (fp8.cu:272-275).  PTX defines div.full only as
 *   "approximate, <= 2 ulp", but on B200 it was compared with amax * fl(1/448)
 *   over every positive float and the two agree bit for bit (2 139 095 040 of
 *   2 139 095 040 inputs), so that product is what is restated here; the golden
 *   vectors recorded from the reference kernel (tests/golden/ref_quant.npz) pin it.
 *   It differs from the IEEE quotient by 1 ulp on ~59 % of scales.
 * div_mode 0: scale = amax / 448 with IEEE division.
 */
static inline float orc_scale_of_amax(float amax, int div_mode) {
  if (div_mode == 1) {
    const volatile float rcp = 1.0f / 448.0f; /* correctly rounded reciprocal, then one rounded product */
    return amax * rcp;
  }
  return amax / 448.0f;
}

void orc_quant_1x128_mode(const uint16_t* x_bf16, int64_t rows, int64_t cols, uint8_t* q, float* scales,
                          int div_mode) {
  const int64_t groups = cols / 128;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    for (int64_t g = 0; g < groups; g++) {
      const uint16_t* src = x_bf16 + r * cols + g * 128;
      float amax = 0.0f;
      for (int k = 0; k < 128; k++) amax = fmaxf(amax, fabsf(orc_bf16_to_f32(src[k])));
      float scale = orc_scale_of_amax(amax, div_mode);
      scales[r * groups + g] = scale;
      float inv = 1.0f / scale;
      for (int k = 0; k < 128; k++) {
        float v = orc_bf16_to_f32(src[k]) * inv;
        float c = fmaxf(-448.0f, fminf(v, 448.0f));
        q[r * cols + g * 128 + k] = orc_f32_to_e4m3(c);
      }
    }
  }
}

void orc_quant_1x128(const uint16_t* x_bf16, int64_t rows, int64_t cols, uint8_t* q, float* scales) {
  orc_quant_1x128_mode(x_bf16, rows, cols, q, scales, 0);
}

/* quant/fp8.cu:299-330: x = float(code) * scale, rounded to bf16. */
void orc_dequant_1x128(const uint8_t* q, const float* scales, int64_t rows, int64_t cols, uint16_t* x_bf16) {
  const int64_t groups = cols / 128;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++)
      x_bf16[r * cols + c] = orc_f32_to_bf16(orc_e4m3_to_f32(q[r * cols + c]) * scales[r * groups + c / 128]);
}

/*
 * Weight quantisation: one fp32 scale per 128x128 block = amax/448 (the layer
 * contract; the reference ships no block-scaled weight quantiser).  w is
 * [n, k] row-major fp32; scales are [ceil(n/128), ceil(k/128)] row-major.  The
 * arithmetic per element is the same as orc_quant_1x128.
 */
void orc_quant_block128(const float* w, int64_t n, int64_t k, uint8_t* q, float* scales) {
  const int64_t nb = CEILDIV(n, 128), kb = CEILDIV(k, 128);
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < nb; bi++) {
    for (int64_t bj = 0; bj < kb; bj++) {
      int64_t i1 = (bi + 1) * 128 < n ? (bi + 1) * 128 : n;
      int64_t j1 = (bj + 1) * 128 < k ? (bj + 1) * 128 : k;
      float amax = 0.0f;
      for (int64_t i = bi * 128; i < i1; i++)
        for (int64_t j = bj * 128; j < j1; j++) amax = fmaxf(amax, fabsf(w[i * k + j]));
      float scale = amax / 448.0f;
      scales[bi * kb + bj] = scale;
      float inv = 1.0f / scale;
      for (int64_t i = bi * 128; i < i1; i++)
        for (int64_t j = bj * 128; j < j1; j++) {
          float c = fmaxf(-448.0f, fminf(w[i * k + j] * inv, 448.0f));
          q[i * k + j] = orc_f32_to_e4m3(c);
        }
    }
  }
}

/* ------------------------------------------------------------------ S1 dispatch plan */

/*
 * scheduler/comm_expander_ver2.cu:30-172 (+ launcher :174-183).
 * idx[T,k] (negative = zero-computation expert, skipped :71).
 * Out: mapping[<= T*W] = ep*T + src in send order; incl[W*S] inclusive counts.
 * Returns the number of mapping entries written.  NT = clamp(ceil(T/16),1,128).
 */
int orc_comm_plan(const int32_t* idx, int T, int k, int E, int W, int S, int32_t* mapping, int32_t* incl) {
  if (T == 0) { memset(incl, 0, sizeof(int32_t) * W * S); return 0; }
  const int EL = E / W, EPS = EL / S;
  int NT = CEILDIV(T, 16); if (NT > 128) NT = 128; if (NT < 1) NT = 1;
  const int NO_LEAD = -993;
  int32_t* lead = (int32_t*)malloc(sizeof(int32_t) * (size_t)T * W);
  int32_t* sums = (int32_t*)calloc((size_t)(NT + 1) * W * EL, sizeof(int32_t));
#define SUMS(r, ep, e) sums[((size_t)(r) * W + (ep)) * EL + (e)]
  for (int t = 0; t < T; t++) {
    for (int ep = 0; ep < W; ep++) lead[t * W + ep] = NO_LEAD;
    for (int j = 0; j < k; j++) {
      int e = idx[t * k + j];
      if (e < 0) continue;
      int ep = e / EL, le = e % EL;
      int cur = lead[t * W + ep];
      if (cur == NO_LEAD || le < cur) lead[t * W + ep] = le;
    }
  }
  for (int tid = 0; tid < NT; tid++)
    for (int t = tid; t < T; t += NT)
      for (int ep = 0; ep < W; ep++) {
        int le = lead[t * W + ep];
        if (le != NO_LEAD) SUMS(tid + 1, ep, le) += 1;
      }
  for (int ep = 0; ep < W; ep++)
    for (int e = 0; e < EL; e++)
      for (int r = 1; r <= NT; r++) SUMS(r, ep, e) += SUMS(r - 1, ep, e);
  int prev = 0;
  for (int ep = 0; ep < W; ep++)
    for (int s = 0; s < S; s++) {
      int c = 0;
      for (int e = s * EPS; e < (s + 1) * EPS; e++) c += SUMS(NT, ep, e);
      prev += c;
      incl[ep * S + s] = prev;
    }
  {
    int sum = 0;
    int32_t* arr = &SUMS(NT, 0, 0);
    for (int i = 0; i < EL * W; i++) { int c = arr[i]; arr[i] = sum; sum += c; }
  }
  for (int tid = 0; tid < NT; tid++)
    for (int t = tid; t < T; t += NT)
      for (int ep = 0; ep < W; ep++) {
        int le = lead[t * W + ep];
        if (le != NO_LEAD) {
          int base = SUMS(NT, ep, le);
          int off = SUMS(tid, ep, le);
          mapping[base + off] = ep * T + t;
          SUMS(tid, ep, le) = off + 1;
        }
      }
#undef SUMS
  free(lead); free(sums);
  return prev;
}

/* ------------------------------------------------------------------ S2 receive plan */

/*
 * communication/alltoall_runner.cu:60-101.  gathered[W][W*S]: row d is rank
 * d's inclusive send plan.  For my_rank: recv_plan[W*S] = inclusive scan of the
 * counts every device sends to me, ordered (device, stage);
 * remote_recv_plan[rank*S+s] = row offset at which my stage-s block lands in
 * rank's receive buffer.  Returns the total number of rows my_rank receives.
 */
int orc_recv_plan(const int32_t* gathered, int my_rank, int W, int S, int32_t* recv_plan, int32_t* remote_recv_plan) {
  int total = 0;
  for (int rank = 0; rank < W; rank++) {
    int run = 0;
    for (int i = 0; i < W * S; i++) {
      int stage = i % S, dev = i / S;
      int begin = (rank == 0 && stage == 0) ? 0 : gathered[dev * W * S + rank * S + stage - 1];
      int end = gathered[dev * W * S + rank * S + stage];
      int n = end - begin;
      if (dev == my_rank) remote_recv_plan[rank * S + stage] = run; /* exclusive */
      run += n;
      if (rank == my_rank) recv_plan[i] = run;
    }
    if (rank == my_rank) total = run;
  }
  return total;
}

/* ------------------------------------------------------------------ S3 GEMM plan */

/*
 * scheduler/gemm_expander_ver2.cu:31-178 (+ helper :6-29).
 * ridx[R,k]: expert ids of the received rows.  Local experts are [lo, hi).
 * Out: excl[hi-lo+1]; mapping[D] = recv_row*k + slot, grouped by local expert,
 * ordered inside an expert by (thread = row mod NT, row, slot) with
 * NT = min(ceil(max_tok_per_gpu*W/16), 128).  Returns D.
 */
int orc_gemm_plan(const int32_t* ridx, int R, int k, int lo, int hi, int max_tok_per_gpu, int W,
                  int32_t* excl, int32_t* mapping) {
  const int EL = hi - lo;
  int64_t tot = (int64_t)max_tok_per_gpu * W;
  int NT = (int)CEILDIV(tot, 16); if (NT > 128) NT = 128; if (NT < 1) NT = 1;
  int32_t* sums = (int32_t*)calloc((size_t)(NT + 1) * EL, sizeof(int32_t));
#define SUMS(r, e) sums[(size_t)(r) * EL + (e)]
  for (int tid = 0; tid < NT; tid++)
    for (int r = tid; r < R; r += NT)
      for (int j = 0; j < k; j++) {
        int g = ridx[r * k + j];
        if (lo <= g && g < hi) SUMS(tid + 1, g - lo) += 1;
      }
  for (int e = 0; e < EL; e++)
    for (int r = 1; r <= NT; r++) SUMS(r, e) += SUMS(r - 1, e);
  excl[0] = 0;
  int prev = 0;
  for (int e = 0; e < EL; e++) { prev += SUMS(NT, e); excl[e + 1] = prev; }
  for (int e = 0; e < EL; e++) SUMS(NT, e) = excl[e];
  for (int tid = 0; tid < NT; tid++)
    for (int r = tid; r < R; r += NT)
      for (int j = 0; j < k; j++) {
        int g = ridx[r * k + j];
        if (lo <= g && g < hi) {
          int e = g - lo;
          mapping[SUMS(NT, e) + SUMS(tid, e)] = r * k + j;
          SUMS(tid, e) += 1;
        }
      }
#undef SUMS
  free(sums);
  return prev;
}

/* ------------------------------------------------------------------ S4 local-reduce plan */

/*
 * scheduler/local_reducer_ver2.cu:25-243 (the one-thread decode variant
 * :245-469 computes the same thing).  Per source-rank block of received rows
 * (bounds from recv_incl), a stable counting sort by tailing (max) local
 * expert:
 *   scale_map[q] = recv row, red_map[q,k] = GEMM row or the sentinel R*k,
 *   ret_incl[W*S] inclusive by (source rank, stage of the tail).
 * gemm_map/excl are S3's outputs.  R = recv_incl[W*S-1].
 */
void orc_local_reduce_plan(const int32_t* ridx, const int32_t* recv_incl, const int32_t* gemm_map,
                           const int32_t* excl, int k, int lo, int hi, int W, int S,
                           int32_t* scale_map, int32_t* red_map, int32_t* ret_incl) {
  const int EL = hi - lo, EPS = EL / S;
  const int R = recv_incl[W * S - 1];
  const int D = excl[EL];
  int32_t* tail = (int32_t*)malloc(sizeof(int32_t) * (size_t)(R > 0 ? R : 1));
  int32_t* r2q = (int32_t*)malloc(sizeof(int32_t) * (size_t)(R > 0 ? R : 1));
  int32_t* cnt = (int32_t*)malloc(sizeof(int32_t) * (size_t)(EL + 1));
  for (int dp = 0; dp < W; dp++) {
    int start = dp == 0 ? 0 : recv_incl[(dp - 1) * S + S - 1];
    int next = recv_incl[dp * S + S - 1];
    memset(cnt, 0, sizeof(int32_t) * (size_t)(EL + 1));
    for (int r = start; r < next; r++) {
      int t = -1;
      for (int j = 0; j < k; j++) {
        int g = ridx[r * k + j];
        if (lo <= g && g < hi && g - lo > t) t = g - lo;
      }
      tail[r] = t; /* every received row has >= 1 local expert by construction */
      if (t >= 0) cnt[t] += 1;
    }
    for (int s = 0; s < S; s++) {
      int c = 0;
      for (int e = s * EPS; e < (s + 1) * EPS; e++) c += cnt[e];
      ret_incl[dp * S + s] = c;
    }
    int sum = 0;
    for (int e = 0; e < EL; e++) { int c = cnt[e]; cnt[e] = sum; sum += c; }
    for (int r = start; r < next; r++) {
      int t = tail[r];
      if (t < 0) continue;
      int q = start + cnt[t]++;
      scale_map[q] = r;
      r2q[r] = q;
    }
  }
  for (int i = 1; i < W * S; i++) ret_incl[i] += ret_incl[i - 1];
  for (int i = 0; i < R * k; i++) red_map[i] = R * k;
  for (int d = 0; d < D; d++) {
    int m = gemm_map[d];
    red_map[r2q[m / k] * k + m % k] = d;
  }
  free(tail); free(r2q); free(cnt);
}

/* ------------------------------------------------------------------ S5 global-reduce plan */

/*
 * scheduler/global_reducer_ver2.cu:31-204.  On the source rank: per
 * destination block of the send order, a stable counting sort by tailing expert
 * on that destination.  glob_map[t*W+ep] = row of the returned buffer holding
 * token t's partial sum from rank ep, or the sentinel T*W;
 * coll_incl[W*S] inclusive by (destination, stage of the tail).
 */
void orc_global_reduce_plan(const int32_t* idx, const int32_t* send_map, const int32_t* send_incl, int T, int k,
                            int E, int W, int S, int32_t* glob_map, int32_t* coll_incl) {
  if (T == 0) { memset(coll_incl, 0, sizeof(int32_t) * W * S); return; }
  const int EL = E / W, EPS = EL / S;
  for (int i = 0; i < T * W; i++) glob_map[i] = T * W;
  int32_t* cnt = (int32_t*)malloc(sizeof(int32_t) * (size_t)(EL + 1));
  int ntot = send_incl[W * S - 1];
  int32_t* tail = (int32_t*)malloc(sizeof(int32_t) * (size_t)(ntot > 0 ? ntot : 1));
  for (int ep = 0; ep < W; ep++) {
    int b = ep == 0 ? 0 : send_incl[(ep - 1) * S + S - 1];
    int e_ = send_incl[ep * S + S - 1];
    memset(cnt, 0, sizeof(int32_t) * (size_t)(EL + 1));
    for (int i = b; i < e_; i++) {
      int t = send_map[i] % T, tl = -1;
      for (int j = 0; j < k; j++) {
        int g = idx[t * k + j];
        if (g < 0) continue;
        int le = g - ep * EL;
        if (0 <= le && le < EL && le > tl) tl = le;
      }
      tail[i] = tl;
      if (tl >= 0) cnt[tl] += 1;
    }
    for (int s = 0; s < S; s++) {
      int c = 0;
      for (int e = s * EPS; e < (s + 1) * EPS; e++) c += cnt[e];
      coll_incl[ep * S + s] = c;
    }
    int sum = 0;
    for (int e = 0; e < EL; e++) { int c = cnt[e]; cnt[e] = sum; sum += c; }
    for (int i = b; i < e_; i++) {
      int tl = tail[i];
      if (tl < 0) continue;
      int t = send_map[i] % T;
      glob_map[t * W + ep] = b + cnt[tl]++;
    }
  }
  for (int i = 1; i < W * S; i++) coll_incl[i] += coll_incl[i - 1];
  free(cnt); free(tail);
}

/* ------------------------------------------------------------------ S6 zero-expert plan */

/* scheduler/zero_reducer.cu:11-25: zero_scale[t] = sum over slots with idx<0 of w, in slot order (fp32). */
void orc_zero_plan(const int32_t* idx, const float* w, int T, int k, float* zero_scale) {
  for (int t = 0; t < T; t++) {
    float s = 0.0f;
    for (int j = 0; j < k; j++)
      if (idx[t * k + j] < 0) s += w[t * k + j];
    zero_scale[t] = s;
  }
}

/* ------------------------------------------------------------------ F1 / F2 fast_ep plans */

/*
 * fast_ep/all_to_all/fast_ep_kernels.cu:105-156 (serial variant; :40-103 is
 * the warp-scan variant with the same result).  excl[E+1] over GLOBAL experts;
 * mapping[i] for slot i=t*k+j: zero-computation slots get t + 1000000 (:16,
 * :84-91); others get slots handed out from the END of the expert's range in
 * ascending i (:93-102), so rows of one expert are in descending i.
 */
void orc_fastep_expand_plan(const int32_t* idx, int T, int k, int E, int32_t* excl, int32_t* mapping) {
  int32_t* cnt = (int32_t*)calloc((size_t)E + 1, sizeof(int32_t));
  for (int i = 0; i < T * k; i++) if (idx[i] >= 0) cnt[idx[i]] += 1;
  int acc = 0;
  excl[0] = 0;
  for (int e = 0; e < E; e++) { acc += cnt[e]; cnt[e] = acc; excl[e + 1] = acc; }
  for (int i = 0; i < T * k; i++) {
    int e = idx[i];
    if (e < 0) mapping[i] = i / k + 1000000;
    else { mapping[i] = cnt[e] - 1; cnt[e] -= 1; }
  }
  free(cnt);
}

/*
 * fast_ep_kernels.cu:510-589 (blockAllGatherPlanKernel; planKernel<N> :490-508
 * is the warp version).  all_gathered[W][E+1] = every rank's excl.
 * Out for my_rank: remote_recv_plan[W], local_send_plan[W+1], gemm_plan[EL+1],
 * arrange src/rows/dst [EL*W] indexed [local_expert*W + src_rank].
 */
void orc_fastep_plan(const int32_t* all_gathered, int my_rank, int W, int E, int32_t* remote_recv_plan,
                     int32_t* local_send_plan, int32_t* gemm_plan, int32_t* arr_src, int32_t* arr_rows,
                     int32_t* arr_dst) {
  const int EL = E / W;
  for (int i = 0; i < W; i++) {
    int v = 0;
    for (int j = 0; j < my_rank; j++) {
      const int32_t* ex = all_gathered + (size_t)(E + 1) * j;
      v += ex[(i + 1) * EL] - ex[i * EL];
    }
    remote_recv_plan[i] = v;
  }
  int acc = 0;
  local_send_plan[0] = 0;
  for (int i = 0; i < W; i++) {
    const int32_t* ex = all_gathered + (size_t)(E + 1) * i;
    acc += ex[(my_rank + 1) * EL] - ex[my_rank * EL];
    local_send_plan[i + 1] = acc;
  }
  acc = 0;
  gemm_plan[0] = 0;
  for (int i = 0; i < EL; i++) {
    for (int j = 0; j < W; j++) {
      int pos = (E + 1) * j + my_rank * EL + i;
      arr_dst[i * W + j] = acc;
      acc += all_gathered[pos + 1] - all_gathered[pos];
    }
    gemm_plan[i + 1] = acc;
  }
  acc = 0;
  for (int j = 0; j < W; j++)
    for (int i = 0; i < EL; i++) {
      int pos = (E + 1) * j + my_rank * EL + i;
      int rows = all_gathered[pos + 1] - all_gathered[pos];
      arr_src[i * W + j] = acc;
      arr_rows[i * W + j] = rows;
      acc += rows;
    }
}

/* ------------------------------------------------------------------ GEMM / SwiGLU / reduce */

/*
 * Block-scaled grouped GEMM in fp32 on dequantised operands (the layer's
 * numerical standard; replaces executor/aok_grouped_gemm.cu:22-37 ->
 * gemm/.../hopper_grouped_gemm_kernel.h:322-400, alpha=1 beta=0 fp32
 * accumulate).  For expert e, rows [excl[e], excl[e+1]):
 *   C[m,n] = sum_kb a_s[m,kb] * b_s[e, n/128, kb] * sum_{k in kb} A[m,k] * B[e,n,k]
 * A: [D,K] e4m3 codes, a_s: [D,K/128]; B: [E,N,K] codes, b_s: [E,ceil(N/128),K/128].
 * C: [D,N] fp32.
 */
void orc_grouped_gemm_fp8(const uint8_t* A, const float* a_s, const uint8_t* B, const float* b_s,
                          const int32_t* excl, int E, int64_t N, int64_t K, float* C) {
  float lut[256];
  orc_e4m3_table(lut);
  const int64_t KB = K / 128, NB = CEILDIV(N, 128);
  for (int e = 0; e < E; e++) {
    const int m0 = excl[e], m1 = excl[e + 1];
    if (m1 <= m0) continue;
    const int64_t rows = m1 - m0;
    float* af = (float*)malloc(sizeof(float) * (size_t)rows * K); /* dequantised codes (scales applied later) */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows * K; i++) af[i] = lut[A[(size_t)m0 * K + i]];
#pragma omp parallel
    {
      float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
      for (int64_t n = 0; n < N; n++) {
        const uint8_t* bp = B + ((size_t)e * N + n) * K;
        const float* bs = b_s + ((size_t)e * NB + n / 128) * KB;
        for (int64_t kk = 0; kk < K; kk++) wrow[kk] = lut[bp[kk]];
        for (int64_t m = 0; m < rows; m++) {
          const float* ap = af + (size_t)m * K;
          const float* as = a_s + (size_t)(m0 + m) * KB;
          float acc = 0.0f;
          for (int64_t kb = 0; kb < KB; kb++) {
            /* 16 interleaved partial sums, reduced in a fixed order: vectorisable and deterministic */
            float ps[16];
            for (int j = 0; j < 16; j++) ps[j] = 0.0f;
            const float* a8 = ap + kb * 128;
            const float* w8 = wrow + kb * 128;
            for (int t = 0; t < 128; t += 16)
              for (int j = 0; j < 16; j++) ps[j] += a8[t + j] * w8[t + j];
            float part = 0.0f;
            for (int j = 0; j < 16; j++) part += ps[j];
            acc += (as[kb] * bs[kb]) * part;
          }
          C[(size_t)(m0 + m) * N + n] = acc;
        }
      }
      free(wrow);
    }
    free(af);
  }
}

/*
 * SwiGLU on rows of [gate(I) | up(I)] (executor/activations.cu:17-39,
 * common/cuda_utils.cuh:71-90): silu(g) = g / (1 + exp(-g)) in fp32, times up
 * in fp32.  The oracle uses expf where the reference uses __expf; the
 * tolerance of the layer test covers the difference.  Output fp32.
 */
void orc_swiglu(const float* gate_up, int64_t rows, int64_t I, float* act) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int64_t j = 0; j < I; j++) {
      float g = gate_up[r * 2 * I + j], u = gate_up[r * 2 * I + I + j];
      act[r * I + j] = (g / (1.0f + expf(-g))) * u;
    }
}

/* fp32 rows -> e4m3 codes + 1x128 scales (same arithmetic as orc_quant_1x128). */
void orc_quant_1x128_f32(const float* x, int64_t rows, int64_t cols, uint8_t* q, float* scales) {
  const int64_t groups = cols / 128;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int64_t g = 0; g < groups; g++) {
      const float* src = x + r * cols + g * 128;
      float amax = 0.0f;
      for (int k = 0; k < 128; k++) amax = fmaxf(amax, fabsf(src[k]));
      float scale = amax / 448.0f;
      scales[r * groups + g] = scale;
      float inv = 1.0f / scale;
      for (int k = 0; k < 128; k++)
        q[r * cols + g * 128 + k] = orc_f32_to_e4m3(fmaxf(-448.0f, fminf(src[k] * inv, 448.0f)));
    }
}

/*
 * fast_ep combine (fast_ep_kernels.cu:231-335): out[t,:] = bf16( sum_j
 * w[t,j] * row(mapping[t*k+j]) [+ shared[t,:]] ), fp32 accumulation in slot
 * order as fused multiply-adds; a mapping >= 1000000 reads the raw input
 * token (identity expert, :282-287).
 */
void orc_fastep_reduce(const uint16_t* rows_bf16, const uint16_t* raw_bf16, const uint16_t* shared_bf16,
                       const float* w, const int32_t* mapping, int T, int k, int64_t H, uint16_t* out_bf16) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++)
    for (int64_t h = 0; h < H; h++) {
      float acc = 0.0f;
      for (int j = 0; j < k; j++) {
        int m = mapping[t * k + j];
        const uint16_t* src = m >= 1000000 ? raw_bf16 + (size_t)(m - 1000000) * H : rows_bf16 + (size_t)m * H;
        acc = fmaf(orc_bf16_to_f32(src[h]), w[t * k + j], acc);
      }
      if (shared_bf16) acc += orc_bf16_to_f32(shared_bf16[(size_t)t * H + h]);
      out_bf16[(size_t)t * H + h] = orc_f32_to_bf16(acc);
    }
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n > 0 ? n : 1);
#else
  (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
