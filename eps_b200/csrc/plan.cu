// Index plans of the EPS scheduler and of fast_ep, for sm_100a.
//
// Every plan of the reference is a stable counting sort whose visiting order is
// an artefact of a strided single-CTA thread decomposition.  Here each plan is
// a thread-block cluster of 1 to 8 CTAs of 32 warps running the same primitive:
// the positions are put in the reference's visiting order ("virtual order"), cut
// into one contiguous range per warp of the cluster, counted per warp with
// warp-match votes (no atomics), scanned over warps, over the cluster's CTAs
// (each CTA reads the others' bucket totals through distributed shared memory)
// and over buckets, and emitted by rank.  The outputs are bit-identical to the
// reference's, including for inputs that repeat an expert id inside a token.
#include <cooperative_groups.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace epsb {

namespace {

constexpr int kPlanThreads = 1024;
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kMaxBuckets = 1024;

constexpr int kMaxCluster = 8;  // portable cluster size
constexpr int kPlanStatusRowsExceeded = EPSB_PLAN_ROWS_EXCEEDED;

struct SortScratch {
  int32_t* rows;    // [kPlanWarps][B] per-warp counts, then per-warp exclusive offsets inside this CTA
  int32_t* base;    // [B] exclusive scan of the bucket totals (whole cluster)
  int32_t* total;   // [B] bucket totals of the whole cluster
  int32_t* ltotal;  // [B] bucket totals of this CTA; the other CTAs of the cluster read it
  int32_t* cbase;   // [B] sum of the totals of the CTAs before this one
  int32_t* wsum;    // [kPlanWarps + 1]
};

constexpr int kScratchRows = kPlanWarps + 4;

__device__ __forceinline__ SortScratch carve(int32_t* smem, int B) {
  SortScratch s;
  s.rows = smem;
  s.base = smem + kPlanWarps * B;
  s.total = s.base + B;
  s.ltotal = s.total + B;
  s.cbase = s.ltotal + B;
  s.wsum = s.cbase + B;
  return s;
}

size_t sort_smem_bytes(int B) { return sizeof(int32_t) * ((size_t)kScratchRows * B + kPlanWarps + 2); }

// CTAs per plan: one per 1024 items, a power of two up to the portable cluster size or the caller's limit
// (max_cluster 0 = no limit of the caller's).
int cluster_size_for(int64_t n_items, int max_cluster = 0) {
  const int limit = max_cluster > 0 && max_cluster < kMaxCluster ? max_cluster : kMaxCluster;
  int c = 1;
  while (c * 2 <= limit && (int64_t)c * kPlanThreads < n_items) c *= 2;
  return c;
}
// Items one CTA of a c-CTA cluster owns (what its key cache has to hold).
int64_t cta_items(int64_t n_items, int c) {
  const int64_t per_warp = ((n_items + (int64_t)c * kPlanThreads - 1) / ((int64_t)c * kPlanThreads)) * 32;
  return per_warp * kPlanWarps;
}

// Shared memory left for the key cache (uint16 per item) after the scratch of a B-bucket sort.
constexpr size_t kPlanSmemBudget = 200 * 1024;
size_t key_cache_bytes(int B, int64_t n_items) {
  const size_t need = ((size_t)n_items * 2 + 15) & ~(size_t)15;
  const size_t used = sort_smem_bytes(B);
  return used + need <= kPlanSmemBudget ? need : 0;
}
__device__ __forceinline__ uint16_t* cache_after(int32_t* smem, int B, int cache_items) {
  if (cache_items <= 0) return nullptr;
  return reinterpret_cast<uint16_t*>(smem + kScratchRows * B + kPlanWarps + 2);
}

// Inclusive scan of one value per thread over the whole 1024-thread CTA.
__device__ __forceinline__ int block_inclusive_scan(int v, int32_t* wsum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, v, off);
    if (lane >= off) v += n;
  }
  __syncthreads();  // wsum may still be read by a previous scan
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = wsum[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += n;
    }
    wsum[lane] = w;
  }
  __syncthreads();
  if (warp > 0) v += wsum[warp - 1];
  return v;
}

// Position `v` of the reference's visiting order -> element index, when NT
// threads each walk elements tid, tid+NT, tid+2NT, ... of n elements.
__device__ __forceinline__ int strided_order(int v, int n, int NT) {
  const int q = n / NT, r = n % NT;
  int tid, i;
  if (v < r * (q + 1)) {
    tid = v / (q + 1);
    i = v % (q + 1);
  } else {
    const int vv = v - r * (q + 1);
    tid = r + vv / q;
    i = vv % q;
  }
  return tid + i * NT;
}

// The sort primitive.  P provides:
//   int  slots()                       sub-items per position
//   int  key(int pos, int j)           bucket of sub-item j of position pos, or -1
//   void emit(int pos, int j, int out) called once per sub-item with key >= 0
//   void skip(int pos, int j)          called once per sub-item with key < 0
// Positions 0..n_pos-1 are already in visiting order.  On return s.base/s.total
// hold the exclusive bucket offsets and the bucket sizes.
template <class P>
__device__ void stable_bucket_sort(P& p, int n_pos, int B, SortScratch s, uint16_t* key_cache = nullptr) {
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned lt_mask = (1u << lane) - 1u;
  // Items (position, slot) are numbered position-major; a warp owns a contiguous range of items and
  // visits it 32 at a time, so the lane order inside a step is the visiting order; warps are numbered
  // through the cluster (CTA-major).  Keys of kKeyUnroll steps are fetched together (independent global
  // loads in flight) and, when the caller provides room, cached in shared memory (indexed from the CTA's
  // first item) so that the emission pass does not touch global memory for them again.
  constexpr int kKeyUnroll = 4;
  const int J = p.slots();
  const int n_items = n_pos * J;
  const int chunk = ((n_items + C * kPlanThreads - 1) / (C * kPlanThreads)) * 32;
  const int cta_begin = min(n_items, crank * kPlanWarps * chunk);
  const int i_begin = min(n_items, (crank * kPlanWarps + warp) * chunk), i_end = min(n_items, i_begin + chunk);
  for (int i = threadIdx.x; i < kPlanWarps * B; i += kPlanThreads) s.rows[i] = 0;
  __syncthreads();
  int32_t* my_row = s.rows + warp * B;
  for (int i0 = i_begin; i0 < i_end; i0 += 32 * kKeyUnroll) {
    int keys[kKeyUnroll];
#pragma unroll
    for (int u = 0; u < kKeyUnroll; u++) {
      const int i = i0 + u * 32 + lane;
      keys[u] = i < i_end ? p.key(i / J, i % J) : -1;
    }
#pragma unroll
    for (int u = 0; u < kKeyUnroll; u++) {
      const int i = i0 + u * 32 + lane;
      if (i0 + u * 32 < i_end) {  // warp-uniform
        const int key = keys[u];
        if (key_cache != nullptr && i < i_end) key_cache[i - cta_begin] = (uint16_t)key;  // -1 -> 0xffff
        const unsigned m = __match_any_sync(0xffffffffu, key);
        if (key >= 0 && (m & lt_mask) == 0) my_row[key] += __popc(m);
        __syncwarp();
      }
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += kPlanThreads) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < kPlanWarps; w++) {
      const int c = s.rows[w * B + b];
      s.rows[w * B + b] = run;
      run += c;
    }
    s.ltotal[b] = run;
  }
  cluster.sync();  // every CTA's bucket totals are in its shared memory
  for (int b = threadIdx.x; b < B; b += kPlanThreads) {
    int before = 0, all = 0;
    for (int c = 0; c < C; c++) {
      const int v = c == crank ? s.ltotal[b] : cluster.map_shared_rank(s.ltotal, c)[b];
      if (c < crank) before += v;
      all += v;
    }
    s.cbase[b] = before;
    s.total[b] = all;
  }
  __syncthreads();
  {
    const int v = threadIdx.x < B ? s.total[threadIdx.x] : 0;
    const int inc = block_inclusive_scan(v, s.wsum);
    if (threadIdx.x < B) s.base[threadIdx.x] = inc - v;
  }
  __syncthreads();
  for (int i0 = i_begin; i0 < i_end; i0 += 32 * kKeyUnroll) {
    int keys[kKeyUnroll];
#pragma unroll
    for (int u = 0; u < kKeyUnroll; u++) {
      const int i = i0 + u * 32 + lane;
      if (i >= i_end) keys[u] = -1;
      else if (key_cache != nullptr) keys[u] = key_cache[i - cta_begin] == 0xffffu ? -1 : (int)key_cache[i - cta_begin];
      else keys[u] = p.key(i / J, i % J);
    }
#pragma unroll
    for (int u = 0; u < kKeyUnroll; u++) {
      const int i = i0 + u * 32 + lane;
      if (i0 + u * 32 < i_end) {  // warp-uniform
        const int key = keys[u];
        const unsigned m = __match_any_sync(0xffffffffu, key);
        int mine = 0;
        if (key >= 0) mine = s.base[key] + s.cbase[key] + my_row[key] + __popc(m & lt_mask);
        __syncwarp();
        if (key >= 0 && (m & lt_mask) == 0) my_row[key] += __popc(m);
        __syncwarp();
        if (i < i_end) {
          if (key >= 0) p.emit(i / J, i % J, mine);
          else p.skip(i / J, i % J);
        }
      }
    }
  }
  // What the CTAs emitted to global memory is visible to the whole cluster, and nobody reads this CTA's
  // bucket totals any more, once every CTA is past this point.
  __threadfence();
  cluster.sync();
}

// Thread index and thread count of the whole cluster, for the element-wise loops around the sorts.
__device__ __forceinline__ int cluster_tid() { return (int)cg::this_cluster().block_rank() * kPlanThreads + threadIdx.x; }
__device__ __forceinline__ int cluster_threads() { return (int)cg::this_cluster().num_blocks() * kPlanThreads; }
__device__ __forceinline__ bool cluster_leader() { return cg::this_cluster().block_rank() == 0; }

// Inclusive count at the end of every (group, stage) run of buckets.
__device__ __forceinline__ void write_stage_sums(const SortScratch& s, int groups, int EL, int S, int32_t* out) {
  const int EPS = EL / S;
  if (!cluster_leader()) return;
  for (int i = threadIdx.x; i < groups * S; i += kPlanThreads) {
    const int g = i / S, st = i % S;
    const int last = g * EL + (st + 1) * EPS - 1;
    out[i] = s.base[last] + s.total[last];
  }
}

// ------------------------------------------------------------------ source side: S1 + S5 + S6

struct CommPlanProblem {
  const int32_t* idx;
  int32_t* send_map;
  int T, k, W, EL, NT;
  __device__ int slots() const { return W; }
  __device__ int token(int pos) const { return strided_order(pos, T, NT); }
  __device__ int key(int pos, int ep) const {
    const int32_t* row = idx + (size_t)token(pos) * k;
    int lead = INT32_MAX;
    for (int j = 0; j < k; j++) {
      const int e = row[j];
      if (e >= 0 && e / EL == ep) lead = min(lead, e % EL);
    }
    return lead == INT32_MAX ? -1 : ep * EL + lead;
  }
  __device__ void emit(int pos, int ep, int out) const { send_map[out] = ep * T + token(pos); }
  __device__ void skip(int, int) const {}
};

struct GlobalPlanProblem {
  const int32_t* idx;
  const int32_t* send_map;
  int32_t* glob_map;
  int T, k, W, EL;
  __device__ int slots() const { return 1; }
  __device__ int key(int pos, int) const {
    const int m = send_map[pos];
    const int ep = m / T, t = m % T;
    const int32_t* row = idx + (size_t)t * k;
    int tail = -1;
    for (int j = 0; j < k; j++) {
      const int e = row[j];
      if (e >= 0 && e / EL == ep) tail = max(tail, e % EL);
    }
    return tail < 0 ? -1 : ep * EL + tail;
  }
  __device__ void emit(int pos, int, int out) const {
    const int m = send_map[pos];
    glob_map[(size_t)(m % T) * W + m / T] = out;
  }
  __device__ void skip(int, int) const {}
};

__global__ void __launch_bounds__(kPlanThreads, 1)
source_plans_kernel(const int32_t* __restrict__ idx, const float* __restrict__ weights, int T, int k, int E, int W,
                    int S, int32_t* send_map, int32_t* send_incl, int32_t* glob_map, int32_t* coll_incl,
                    float* zero_scale, int cache_items) {
  extern __shared__ int32_t plan_smem[];
  const int EL = E / W;
  SortScratch s = carve(plan_smem, E);
  uint16_t* cache = cache_after(plan_smem, E, cache_items);
  if (zero_scale != nullptr && weights != nullptr) {
    for (int t = cluster_tid(); t < T; t += cluster_threads()) {
      float z = 0.0f;
      for (int j = 0; j < k; j++)
        if (idx[(size_t)t * k + j] < 0) z += weights[(size_t)t * k + j];
      zero_scale[t] = z;
    }
  }
  int NT = (T + 15) / 16;
  NT = max(1, min(NT, 128));
  CommPlanProblem cp{idx, send_map, T, k, W, EL, NT};
  stable_bucket_sort(cp, T, E, s, cache);
  write_stage_sums(s, W, EL, S, send_incl);
  if (glob_map == nullptr) return;
  const int n_sent = s.base[E - 1] + s.total[E - 1];
  for (int i = cluster_tid(); i < T * W; i += cluster_threads()) glob_map[i] = T * W;
  __threadfence();
  cg::this_cluster().sync();  // the glob_map fill (and, from the sort above, send_map) is visible to the cluster
  GlobalPlanProblem gp{idx, send_map, glob_map, T, k, W, EL};
  stable_bucket_sort(gp, n_sent, E, s, cache);
  write_stage_sums(s, W, EL, S, coll_incl);
}

// ------------------------------------------------------------------ S6 alone (callers that plan the sends first)

__global__ void zero_plan_kernel(const int32_t* __restrict__ idx, const float* __restrict__ weights, int T, int k,
                                 float* __restrict__ zero_scale) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    float z = 0.0f;
    for (int j = 0; j < k; j++)
      if (idx[(size_t)t * k + j] < 0) z += weights[(size_t)t * k + j];
    zero_scale[t] = z;
  }
}

// ------------------------------------------------------------------ S2 receive plan

__global__ void __launch_bounds__(kPlanThreads, 1)
recv_plan_kernel(const int32_t* __restrict__ gathered, int my_rank, int W, int S, int32_t* recv_incl,
                 int32_t* remote_offset, int32_t* total_rows) {
  __shared__ int32_t wsum[kPlanWarps + 1];
  const int n = W * S;
  const int i = threadIdx.x;
  for (int rank = 0; rank < W; rank++) {
    int cnt = 0;
    if (i < n) {
      const int stage = i % S, dev = i / S;
      const int begin = (rank == 0 && stage == 0) ? 0 : gathered[(size_t)dev * n + rank * S + stage - 1];
      cnt = gathered[(size_t)dev * n + rank * S + stage] - begin;
    }
    const int inc = block_inclusive_scan(cnt, wsum);
    if (i < n) {
      if (rank == my_rank) {
        recv_incl[i] = inc;
        if (i == n - 1 && total_rows != nullptr) *total_rows = inc;
      }
      if (i / S == my_rank) remote_offset[rank * S + i % S] = inc - cnt;
    }
  }
}

// ------------------------------------------------------------------ expert side: S3 + S4

struct GemmPlanProblem {
  const int32_t* ridx;
  int32_t* gemm_map;
  int32_t* inv_gemm;
  int R, k, lo, hi, NT;
  __device__ int slots() const { return k; }
  __device__ int row(int pos) const { return strided_order(pos, R, NT); }
  __device__ int key(int pos, int j) const {
    const int g = ridx[(size_t)row(pos) * k + j];
    return (lo <= g && g < hi) ? g - lo : -1;
  }
  __device__ void emit(int pos, int j, int out) const {
    const int m = row(pos) * k + j;
    gemm_map[out] = m;
    inv_gemm[m] = out;
  }
  __device__ void skip(int pos, int j) const { inv_gemm[row(pos) * k + j] = R * k; }
};

struct LocalReducePlanProblem {
  const int32_t* ridx;
  const int32_t* recv_incl;
  const int32_t* inv_gemm;
  int32_t* scale_map;
  int32_t* red_map;
  int k, lo, hi, W, S, EL;
  __device__ int slots() const { return 1; }
  __device__ int key(int r, int) const {
    int dp = 0;
    while (dp < W - 1 && r >= recv_incl[dp * S + S - 1]) dp++;
    int tail = -1;
    for (int j = 0; j < k; j++) {
      const int g = ridx[(size_t)r * k + j];
      if (lo <= g && g < hi) tail = max(tail, g - lo);
    }
    return tail < 0 ? -1 : dp * EL + tail;
  }
  __device__ void emit(int r, int, int out) const {
    scale_map[out] = r;
    for (int j = 0; j < k; j++) red_map[(size_t)out * k + j] = inv_gemm[(size_t)r * k + j];
  }
  __device__ void skip(int, int) const {}
};

__global__ void __launch_bounds__(kPlanThreads, 1)
expert_plans_kernel(const int32_t* __restrict__ ridx, const int32_t* __restrict__ recv_incl, int k, int lo, int hi,
                    int W, int S, int NT, int32_t* excl, int32_t* gemm_map, int32_t* inv_gemm, int32_t* scale_map,
                    int32_t* red_map, int32_t* ret_incl, int cache_items, int max_rows, int32_t* status) {
  extern __shared__ int32_t plan_smem[];
  const int EL = hi - lo;
  const int R = recv_incl[W * S - 1];
  // Every buffer, the shared-memory key cache and the cluster size were sized by the host from max_rows.  A row
  // count beyond that promise (a corrupted or foreign receive plan) must not be followed: every CTA takes this
  // same branch, the plans come out empty (no GEMM rows, nothing returned) and the caller's status word says why.
  if (R < 0 || R > max_rows) {
    if (cluster_leader()) {
      for (int e = threadIdx.x; e <= EL; e += kPlanThreads) excl[e] = 0;
      if (ret_incl != nullptr)
        for (int i = threadIdx.x; i < W * S; i += kPlanThreads) ret_incl[i] = 0;
      if (threadIdx.x == 0 && status != nullptr) {
        status[0] = kPlanStatusRowsExceeded;
        status[1] = R;
      }
    }
    return;
  }
  // the cache sits behind the larger of the two scratch layouts so that both sorts can use it
  uint16_t* cache = cache_after(plan_smem, scale_map != nullptr ? W * EL : EL, cache_items);
  {
    SortScratch s = carve(plan_smem, EL);
    GemmPlanProblem gp{ridx, gemm_map, inv_gemm, R, k, lo, hi, NT};
    stable_bucket_sort(gp, R, EL, s, cache);
    if (cluster_leader()) {
      for (int e = threadIdx.x; e < EL; e += kPlanThreads) excl[e + 1] = s.base[e] + s.total[e];
      if (threadIdx.x == 0) excl[0] = 0;
    }
  }
  if (scale_map == nullptr) return;
  __syncthreads();  // inv_gemm is complete and visible (the sort ended with a cluster-wide fence and barrier)
  SortScratch s = carve(plan_smem, W * EL);
  LocalReducePlanProblem lp{ridx, recv_incl, inv_gemm, scale_map, red_map, k, lo, hi, W, S, EL};
  stable_bucket_sort(lp, R, W * EL, s, cache);
  write_stage_sums(s, W, EL, S, ret_incl);
}

// ------------------------------------------------------------------ fast_ep: F1, F2

struct FastEpExpandProblem {
  const int32_t* idx;
  int32_t* mapping;
  const int32_t* base;   // shared memory: exclusive offset of every expert
  const int32_t* total;  // shared memory: rows of every expert
  int k;
  __device__ int slots() const { return k; }
  __device__ int key(int t, int j) const {
    const int e = idx[(size_t)t * k + j];
    return e >= 0 ? e : -1;
  }
  // `out` = base + ascending rank; the reference hands slots out from the end of the expert's range.
  __device__ void emit(int t, int j, int out) const {
    const int e = idx[(size_t)t * k + j];
    mapping[(size_t)t * k + j] = base[e] + total[e] - 1 - (out - base[e]);
  }
  __device__ void skip(int t, int j) const { mapping[(size_t)t * k + j] = t + kZcMark; }
};

__global__ void __launch_bounds__(kPlanThreads, 1)
fastep_expand_plan_kernel(const int32_t* __restrict__ idx, int T, int k, int E, int32_t* excl, int32_t* mapping) {
  extern __shared__ int32_t plan_smem[];
  SortScratch s = carve(plan_smem, E);
  FastEpExpandProblem fp{idx, mapping, s.base, s.total, k};
  stable_bucket_sort(fp, T, E, s);
  if (!cluster_leader()) return;
  for (int e = threadIdx.x; e < E; e += kPlanThreads) excl[e + 1] = s.base[e] + s.total[e];
  if (threadIdx.x == 0) excl[0] = 0;
}

__global__ void __launch_bounds__(kPlanThreads, 1)
fastep_plan_kernel(const int32_t* __restrict__ ag, int my_rank, int W, int E, int32_t* remote_recv_plan,
                   int32_t* local_send_plan, int32_t* gemm_plan, int32_t* arr_src, int32_t* arr_rows,
                   int32_t* arr_dst) {
  __shared__ int32_t wsum[kPlanWarps + 1];
  const int EL = E / W;
  const int tid = threadIdx.x;
  const size_t stride = (size_t)E + 1;
  // rows each source rank sends to each of my local experts: index (i = local expert, j = source rank)
  // expert-major order p = i*W + j gives arr_dst / gemm_plan; source-major order gives arr_src.
  {
    const int i = tid / W, j = tid % W;
    int rows = 0;
    if (tid < EL * W) {
      const size_t pos = stride * j + (size_t)my_rank * EL + i;
      rows = ag[pos + 1] - ag[pos];
    }
    const int inc = block_inclusive_scan(rows, wsum);
    if (tid < EL * W) {
      arr_dst[tid] = inc - rows;
      arr_rows[tid] = rows;
      if (j == W - 1) gemm_plan[i + 1] = inc;
    }
    if (tid == 0) gemm_plan[0] = 0;
  }
  {
    const int j = tid / EL, i = tid % EL;
    int rows = 0;
    if (tid < EL * W) {
      const size_t pos = stride * j + (size_t)my_rank * EL + i;
      rows = ag[pos + 1] - ag[pos];
    }
    const int inc = block_inclusive_scan(rows, wsum);
    if (tid < EL * W) {
      arr_src[i * W + j] = inc - rows;
      if (i == EL - 1) local_send_plan[j + 1] = inc;
    }
    if (tid == 0) local_send_plan[0] = 0;
  }
  if (tid < W) {
    int v = 0;
    for (int j = 0; j < my_rank; j++) v += ag[stride * j + (size_t)(tid + 1) * EL] - ag[stride * j + (size_t)tid * EL];
    remote_recv_plan[tid] = v;
  }
}

// ------------------------------------------------------------------ fast_oep: ids grouped by owner rank

struct OepArrangeProblem {
  const int32_t* ids;
  int32_t* mapping;
  int32_t* send_map;
  int32_t size_per_rank;
  int W;
  __device__ int slots() const { return 1; }
  __device__ int key(int i, int) const {
    const int id = ids[i];
    if (id < 0) return -1;
    const int r = id / size_per_rank;
    return r < W ? r : -1;
  }
  __device__ void emit(int i, int, int out) const {
    mapping[i] = out;
    send_map[out] = i;
  }
  __device__ void skip(int i, int) const { mapping[i] = -1; }
};

__global__ void __launch_bounds__(kPlanThreads, 1)
oep_arrange_plan_kernel(const int32_t* __restrict__ ids, int n, int32_t size_per_rank, int W, int32_t* send_incl,
                        int32_t* mapping, int32_t* send_map) {
  extern __shared__ int32_t plan_smem[];
  SortScratch s = carve(plan_smem, W);
  OepArrangeProblem op{ids, mapping, send_map, size_per_rank, W};
  stable_bucket_sort(op, n, W, s);
  if (!cluster_leader()) return;
  for (int r = threadIdx.x; r < W; r += kPlanThreads) send_incl[r] = s.base[r] + s.total[r];
}

// ---------------------------------------------------------------- scratch that nobody has to allocate

// Backing store of epsb_expert_plans_noalloc: the inverse GEMM map (one int32 per received (row, slot)).
// It lives in the library's device image, so every GPU that loads the library holds these 4 MiB until exit.
constexpr int64_t kStaticScratchItems = 1 << 20;
static __device__ __align__(256) int32_t g_inv_gemm_scratch[kStaticScratchItems];

// Device address of the array on the CURRENT device.  In host code the array's name is only a handle: the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device with that device current.
int static_inv_gemm_scratch(int32_t** out) {
  static std::mutex mu;
  static int32_t* per_device[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(EPSB_ERR_INVALID, "device ordinal %d is outside the table of 64", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    int32_t* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_inv_gemm_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(EPSB_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    per_device[dev] = p;
  }
  *out = per_device[dev];
  return EPSB_OK;
}

// Launch of a plan kernel as one cluster of `c` CTAs.
template <class... KArgs, class... Args>
int launch_cluster(void (*kernel)(KArgs...), int c, size_t smem, cudaStream_t st, const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)c, 1, 1);
  cfg.blockDim = dim3(kPlanThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

int set_smem(const void* fn, size_t bytes) {
  if (bytes > 227 * 1024) return fail(EPSB_ERR_INVALID, "plan needs %zu bytes of shared memory (> 227 KB)", bytes);
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  return EPSB_OK;
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_source_plans(const int32_t* idx, const float* weights, int T, int k, int E, int W, int S,
                                 int32_t* send_map, int32_t* send_incl, int32_t* glob_map, int32_t* coll_incl,
                                 float* zero_scale, int max_cluster, void* stream) {
  EPSB_REQUIRE(max_cluster == 0 || max_cluster == 1 || max_cluster == 2 || max_cluster == 4 || max_cluster == 8,
               EPSB_ERR_INVALID, "max_cluster %d is not 0, 1, 2, 4 or 8", max_cluster);
  EPSB_REQUIRE(T >= 0 && k > 0 && E > 0 && W > 0 && S > 0, EPSB_ERR_INVALID, "bad sizes T=%d k=%d E=%d W=%d S=%d", T, k,
               E, W, S);
  EPSB_REQUIRE(E % W == 0, EPSB_ERR_INVALID, "num_experts %d is not divisible by ep_world_size %d", E, W);
  EPSB_REQUIRE((E / W) % S == 0, EPSB_ERR_INVALID, "Invalid num_stages: %d for local_num_experts: %d", S, E / W);
  EPSB_REQUIRE(E <= kMaxBuckets, EPSB_ERR_INVALID, "num_experts %d exceeds %d", E, kMaxBuckets);
  EPSB_REQUIRE((glob_map == nullptr) == (coll_incl == nullptr), EPSB_ERR_INVALID,
               "glob_map and coll_incl go together");
  auto st = static_cast<cudaStream_t>(stream);
  if (T == 0) {  // reference: comm_expander_ver2.cu:175-178, global_reducer_ver2.cu:207-210
    cudaMemsetAsync(send_incl, 0, sizeof(int32_t) * W * S, st);
    if (coll_incl) cudaMemsetAsync(coll_incl, 0, sizeof(int32_t) * W * S, st);
    return check_launch("source_plans(T=0)");
  }
  const int c = cluster_size_for((int64_t)T * W, max_cluster);
  const int64_t per_cta = cta_items((int64_t)T * W, c);
  const size_t cache = key_cache_bytes(E, per_cta);
  const size_t smem = sort_smem_bytes(E) + cache;
  int rc = set_smem((const void*)source_plans_kernel, smem);
  if (rc) return rc;
  return launch_cluster(source_plans_kernel, c, smem, st, "source_plans", idx, weights, T, k, E, W, S, send_map,
                        send_incl, glob_map, coll_incl, zero_scale, cache ? (int)per_cta : 0);
}

extern "C" int epsb_zero_plan(const int32_t* idx, const float* weights, int T, int k, float* zero_scale, void* stream) {
  EPSB_REQUIRE(T >= 0 && k > 0, EPSB_ERR_INVALID, "bad sizes T=%d k=%d", T, k);
  if (T == 0) return EPSB_OK;
  int blocks = (T + 255) / 256;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  zero_plan_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(idx, weights, T, k, zero_scale);
  return check_launch("zero_plan");
}

extern "C" int epsb_recv_plan(const int32_t* gathered, int my_rank, int W, int S, int32_t* recv_incl,
                              int32_t* remote_offset, int32_t* total_rows, void* stream) {
  EPSB_REQUIRE(W > 0 && S > 0 && my_rank >= 0 && my_rank < W, EPSB_ERR_INVALID, "bad rank/world %d/%d", my_rank, W);
  EPSB_REQUIRE(W * S <= kPlanThreads, EPSB_ERR_INVALID, "ep_world_size * num_stages is too big.");
  recv_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(gathered, my_rank, W, S, recv_incl,
                                                                              remote_offset, total_rows);
  return check_launch("recv_plan");
}

extern "C" int epsb_expert_plans(const int32_t* ridx, const int32_t* recv_incl, int k, int lo, int hi, int W, int S,
                                 int max_tok_per_gpu, int64_t max_rows, int32_t* excl, int32_t* gemm_map,
                                 int32_t* inv_gemm, int32_t* scale_map, int32_t* red_map, int32_t* ret_incl,
                                 int32_t* status, int max_cluster, void* stream) {
  const int EL = hi - lo;
  EPSB_REQUIRE(max_cluster == 0 || max_cluster == 1 || max_cluster == 2 || max_cluster == 4 || max_cluster == 8,
               EPSB_ERR_INVALID, "max_cluster %d is not 0, 1, 2, 4 or 8", max_cluster);
  EPSB_REQUIRE(EL > 0 && k > 0 && W > 0 && S > 0, EPSB_ERR_INVALID, "bad sizes EL=%d k=%d W=%d S=%d", EL, k, W, S);
  EPSB_REQUIRE(EL % S == 0, EPSB_ERR_INVALID, "Invalid num_stages: %d for local_num_experts: %d", S, EL);
  EPSB_REQUIRE((int64_t)W * EL <= kMaxBuckets, EPSB_ERR_INVALID, "W*EL = %lld exceeds %d", (long long)W * EL,
               kMaxBuckets);
  EPSB_REQUIRE(max_rows * k < (1ll << 31), EPSB_ERR_INVALID, "max_rows*k overflows int32");
  EPSB_REQUIRE((scale_map == nullptr) == (red_map == nullptr) && (scale_map == nullptr) == (ret_incl == nullptr),
               EPSB_ERR_INVALID, "scale_map, red_map and ret_incl go together");
  int64_t tot = (int64_t)max_tok_per_gpu * W;
  int NT = (int)((tot + 15) / 16);
  if (NT > 128) NT = 128;
  if (NT < 1) NT = 1;
  const int Bmax = scale_map ? W * EL : EL;
  const int c = cluster_size_for(max_rows * k, max_cluster);
  const int64_t per_cta = cta_items(max_rows * k, c);
  const size_t cache = key_cache_bytes(Bmax, per_cta);
  const size_t smem = sort_smem_bytes(Bmax) + cache;
  int rc = set_smem((const void*)expert_plans_kernel, smem);
  if (rc) return rc;
  return launch_cluster(expert_plans_kernel, c, smem, static_cast<cudaStream_t>(stream), "expert_plans", ridx,
                        recv_incl, k, lo, hi, W, S, NT, excl, gemm_map, inv_gemm, scale_map, red_map, ret_incl,
                        cache ? (int)per_cta : 0, (int)max_rows, status);
}

extern "C" int epsb_expert_plans_noalloc(const int32_t* ridx, const int32_t* recv_incl, int k, int lo, int hi, int W,
                                         int S, int max_tok_per_gpu, int64_t max_rows, int32_t* excl,
                                         int32_t* gemm_map, int32_t* scale_map, int32_t* red_map, int32_t* ret_incl,
                                         int32_t* status, int max_cluster, void* stream) {
  EPSB_REQUIRE(k > 0 && max_rows >= 0, EPSB_ERR_INVALID, "bad sizes k=%d max_rows=%lld", k, (long long)max_rows);
  EPSB_REQUIRE(max_rows * k <= kStaticScratchItems, EPSB_ERR_WORKSPACE,
               "max_rows * topk = %lld exceeds the built-in scratch of %lld entries; use epsb_expert_plans with a "
               "caller-provided inv_gemm buffer",
               (long long)(max_rows * k), (long long)kStaticScratchItems);
  int32_t* scratch = nullptr;
  int rc = static_inv_gemm_scratch(&scratch);
  if (rc) return rc;
  return epsb_expert_plans(ridx, recv_incl, k, lo, hi, W, S, max_tok_per_gpu, max_rows, excl, gemm_map, scratch,
                           scale_map, red_map, ret_incl, status, max_cluster, stream);
}

extern "C" int epsb_fastep_expand_plan(const int32_t* idx, int T, int k, int E, int32_t* excl, int32_t* mapping,
                                       void* stream) {
  EPSB_REQUIRE(T >= 0 && k > 0 && E > 0 && E <= kMaxBuckets, EPSB_ERR_INVALID, "bad sizes T=%d k=%d E=%d", T, k, E);
  const size_t smem = sort_smem_bytes(E);
  int rc = set_smem((const void*)fastep_expand_plan_kernel, smem);
  if (rc) return rc;
  return launch_cluster(fastep_expand_plan_kernel, cluster_size_for((int64_t)T * k), smem,
                        static_cast<cudaStream_t>(stream), "fastep_expand_plan", idx, T, k, E, excl, mapping);
}

extern "C" int epsb_oep_arrange_plan(const int32_t* ids, int64_t n, int64_t size_per_rank, int W, int32_t* send_incl,
                                     int32_t* mapping, int32_t* send_map, void* stream) {
  EPSB_REQUIRE(n >= 0 && n < (1ll << 31) && size_per_rank > 0 && size_per_rank < (1ll << 31) && W > 0 &&
                   W <= kMaxBuckets,
               EPSB_ERR_INVALID, "bad sizes n=%lld size_per_rank=%lld W=%d", (long long)n, (long long)size_per_rank, W);
  auto st = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    cudaMemsetAsync(send_incl, 0, sizeof(int32_t) * W, st);
    return check_launch("oep_arrange_plan(n=0)");
  }
  const size_t smem = sort_smem_bytes(W);
  int rc = set_smem((const void*)oep_arrange_plan_kernel, smem);
  if (rc) return rc;
  return launch_cluster(oep_arrange_plan_kernel, cluster_size_for(n), smem, st, "oep_arrange_plan", ids, (int)n,
                        (int32_t)size_per_rank, W, send_incl, mapping, send_map);
}

extern "C" int epsb_fastep_plan(const int32_t* all_gathered, int my_rank, int W, int E, int32_t* remote_recv_plan,
                                int32_t* local_send_plan, int32_t* gemm_plan, int32_t* arr_src, int32_t* arr_rows,
                                int32_t* arr_dst, void* stream) {
  EPSB_REQUIRE(W > 0 && E > 0 && E % W == 0 && my_rank >= 0 && my_rank < W, EPSB_ERR_INVALID,
               "bad sizes W=%d E=%d rank=%d", W, E, my_rank);
  EPSB_REQUIRE(E <= kPlanThreads, EPSB_ERR_INVALID, "num_experts %d exceeds %d", E, kPlanThreads);
  fastep_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      all_gathered, my_rank, W, E, remote_recv_plan, local_send_plan, gemm_plan, arr_src, arr_rows, arr_dst);
  return check_launch("fastep_plan");
}
