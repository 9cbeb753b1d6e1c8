// Device-side expert-parallel exchange over peer memory (sm_100a, one NVSwitch box).
//
// Replaces the reference's mscclpp transport: CommBuffs arenas (src/communication/msccl_comm.cu:191-255), the
// plan all-gather with flags (src/communication/alltoall_runner.cu:39-128), the SM-copy all-to-all
// (alltoall_runner.cu:131-256, smChan_put in msccl_comm.cuh:166-183) and, fused with it, expandForComm
// (src/scheduler/comm_expander.cu:118-215) on the way out and localReduce (src/scheduler/local_reducer.cu:103-211)
// on the way back.
//
// Every rank owns one symmetric REGION (CUDA IPC memory mapped by all ranks of the box): plan tables, flag
// words and the receive arenas.  Nothing goes through the host after set-up:
//   publish_plans   every rank stores its two inclusive plans (what it sends, what it collects back) into every
//                   peer's table and then releases a flag there;
//   recv_plans      waits (bounded) for the W flags, then derives the receive plan and, for both directions, the
//                   row offset at which this rank's block lands in each peer's arena;
//   put             permute-on-send: a warp takes a row of the send order, reads the token's row through the
//                   dispatch plan and stores it straight into the destination's arena (ids, gate weights, FP8
//                   row, scales); the last CTA to finish releases a flag at every peer;
//   wait            bounded spin on the W flags of one exchange (the consumer side);
//   local_reduce_put the expert rank's weighted-row reduction writes each return row straight into the source
//                   rank's collect arena, then flags.
// Only peer STORES and flag loads of local memory are used: no loads from peer memory, no TMA, no multicast.
// Flags carry the call's epoch (a counter that only grows), so they are never reset; the tables and the
// dispatch arenas are double-buffered by epoch parity, which is enough because a rank can only be one exchange
// ahead of a peer (it needs that peer's return rows to finish a call).
// Every spin has a time limit after which the kernel records a code in the caller's status words and returns.
#include <cstring>
#include <new>

#include "common.cuh"

namespace epsb {

namespace {

constexpr int kMaxPeers = EPSB_MAX_PEERS;
constexpr int kXThreads = 256;
constexpr int kXWarps = kXThreads / 32;

struct Layout {
  int64_t table_send, table_coll;  // int32 [2][W][W*S]
  int64_t flags;                   // uint32 [slots][W]
  int64_t idx, wts, hidden, scales;  // [2][rows][cols]
  int64_t out;                     // bf16 [rows][H]
  int64_t total;
  int64_t idx_bytes, wts_bytes, hidden_bytes, scales_bytes;  // bytes of ONE parity copy
};

int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

Layout make_layout(int max_tok, int W, int S, int k, int64_t H, int hidden_elem, int scales_dim) {
  Layout l;
  const int64_t rows = (int64_t)(max_tok > 0 ? max_tok : 1) * W;
  const int64_t n = (int64_t)W * S;
  int64_t off = 0;
  l.table_send = off;
  off = align256(off + 2 * W * n * 4);
  l.table_coll = off;
  off = align256(off + 2 * W * n * 4);
  l.flags = off;
  off = align256(off + (int64_t)(2 + 2 * S) * W * 4);
  l.idx_bytes = align256(rows * k * 4);
  l.wts_bytes = align256(rows * k * 4);
  l.hidden_bytes = hidden_elem > 0 ? align256(rows * H * hidden_elem) : 0;   // 0: an exchange of ids and return rows only
  l.scales_bytes = align256(rows * (scales_dim > 0 ? scales_dim : 1) * 4);
  l.idx = off;
  off += 2 * l.idx_bytes;
  l.wts = off;
  off += 2 * l.wts_bytes;
  l.hidden = off;
  off += 2 * l.hidden_bytes;
  l.scales = off;
  off += 2 * l.scales_bytes;
  l.out = off;
  off = align256(off + rows * H * 2);
  l.total = off;
  return l;
}

}  // namespace

}  // namespace epsb

// The handle behind the C ABI.
struct epsb_exchange {
  int rank, W, max_tok, S, k, hidden_elem, scales_dim;
  int64_t H;
  epsb::Layout lay;
  uint8_t* peer[epsb::kMaxPeers];  // every rank's region as mapped into this process
  int32_t* dev;                    // device scratch: [0] CTA counter of put, [1] of local_reduce_put,
                                   // [16 .. 16+n) dispatch offsets, [16+n .. 16+2n) combine offsets, then recv_incl [n]
  int epoch;
};

namespace epsb {

namespace {

struct Peers {
  uint8_t* base[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spins until *flag >= epoch or the limit runs out; false on time-out.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = now_ns();
  while (true) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (now_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}

// ---------------------------------------------------------------- plans

__global__ void __launch_bounds__(1024, 1)
publish_plans_kernel(Peers peers, int64_t off_send, int64_t off_coll, int64_t off_flags, int rank, int W, int n,
                     int n_max, uint32_t epoch, const int32_t* __restrict__ send_incl,
                     const int32_t* __restrict__ coll_incl) {
  // n = W*S entries of this call, n_max = W*S_max the row pitch of the tables
  const int par = (int)(epoch & 1u);
  for (int i = threadIdx.x; i < W * n; i += blockDim.x) {
    const int p = i / n, j = i % n;
    int32_t* ts = reinterpret_cast<int32_t*>(peers.base[p] + off_send) + ((int64_t)par * W + rank) * n_max;
    int32_t* tc = reinterpret_cast<int32_t*>(peers.base[p] + off_coll) + ((int64_t)par * W + rank) * n_max;
    ts[j] = send_incl[j];
    tc[j] = coll_incl[j];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + off_flags) + rank, epoch);  // slot 0 = plans
  }
}

__device__ __forceinline__ int block_scan_1024(int v, int32_t* wsum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, v, off);
    if (lane >= off) v += t;
  }
  __syncthreads();
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = wsum[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += t;
    }
    wsum[lane] = w;
  }
  __syncthreads();
  if (warp > 0) v += wsum[warp - 1];
  return v;
}

// After the W plan flags: recv_incl [n] (inclusive, source-major then stage; reference alltoall_runner.cu:60-101),
// disp_off [n]: where my (dest p, stage s) block starts in p's dispatch arena, comb_off [n]: where the rows I
// return to source p for stage s start in p's collect arena (p's collect plan, entry (me, s), exclusive).
__global__ void __launch_bounds__(1024, 1)
recv_plans_kernel(const uint8_t* my_base, int64_t off_send, int64_t off_coll, int64_t off_flags, int rank, int W,
                  int S, int n_max, uint32_t epoch, uint64_t limit_ns, int max_rows, int32_t* recv_incl,
                  int32_t* disp_off, int32_t* comb_off, int32_t* recv_incl_out, int32_t* status) {
  __shared__ int32_t wsum[33];
  __shared__ int timed_out;
  const int n = W * S;
  const int par = (int)(epoch & 1u);
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(my_base + off_flags) + threadIdx.x;
    if (!wait_flag(f, epoch, limit_ns)) {
      timed_out = 1;
      if (status != nullptr) {
        atomicCAS(status, 0, EPSB_EXCHANGE_TIMEOUT_PLANS);
        atomicExch(status + 1, (int)threadIdx.x);
      }
    }
  }
  __syncthreads();
  const int i = threadIdx.x;
  if (timed_out) {  // nothing is known about the peers: an empty exchange, so that every later kernel is a no-op
    if (i < n) {
      recv_incl[i] = 0;
      disp_off[i] = 0;
      comb_off[i] = 0;
      if (recv_incl_out != nullptr) recv_incl_out[i] = 0;
    }
    return;
  }
  const int32_t* gs = reinterpret_cast<const int32_t*>(my_base + off_send) + (int64_t)par * W * n_max;
  const int32_t* gc = reinterpret_cast<const int32_t*>(my_base + off_coll) + (int64_t)par * W * n_max;
  bool bad = false;
  for (int dest = 0; dest < W; dest++) {
    int cnt = 0;
    if (i < n) {
      const int stage = i % S, src = i / S;
      const int j = dest * S + stage;
      const int begin = j == 0 ? 0 : gs[(int64_t)src * n_max + j - 1];
      cnt = gs[(int64_t)src * n_max + j] - begin;
    }
    const int inc = block_scan_1024(cnt, wsum);
    if (i < n) {
      if (dest == rank) {
        recv_incl[i] = inc;
        if (recv_incl_out != nullptr) recv_incl_out[i] = inc;
        if (i == n - 1 && (inc > max_rows || inc < 0)) bad = true;
      }
      if (i / S == rank) disp_off[dest * S + i % S] = inc - cnt;
    }
  }
  if (i < n) {
    const int p = i / S, s = i % S;
    const int j = rank * S + s;
    comb_off[i] = j == 0 ? 0 : gc[(int64_t)p * n_max + j - 1];
  }
  if (bad && status != nullptr) {  // more rows announced than the arena holds: refuse, like the reference's arena check
    atomicCAS(status, 0, EPSB_EXCHANGE_ROWS_EXCEEDED);
  }
}

// ---------------------------------------------------------------- put (permute-on-send)

struct PutArgs {
  const int32_t* idx;      // [T,k]
  const float* wts;        // [T,k]
  const uint8_t* hidden;   // [T,hidden_row_bytes]
  const float* scales;     // [T,scales_dim]
  const int32_t* send_map; // [<= T*W] = ep*T + token
  const int32_t* send_incl;  // [W*S]
  const int32_t* disp_off;   // [W*S]
  int64_t off_idx, off_wts, off_hidden, off_scales, off_flags;  // region offsets of the CURRENT parity's arenas
  int64_t hidden_row_bytes;
  int T, k, scales_dim, W, S, stage, mask, flag_slot, rank;
  uint32_t epoch;
  int32_t* cta_counter;
};

__device__ __forceinline__ void copy_row16(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int vecs,
                                           int lane) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  int v = lane;
  for (; v + 96 < vecs; v += 128) {
    const uint4 a = ld_nc_16(s + v), b = ld_nc_16(s + v + 32), c = ld_nc_16(s + v + 64), e = ld_nc_16(s + v + 96);
    st_16(d + v, a);
    st_16(d + v + 32, b);
    st_16(d + v + 64, c);
    st_16(d + v + 96, e);
  }
  for (; v < vecs; v += 32) st_16(d + v, ld_nc_16(s + v));
}

// The last CTA of a grid to get here releases `flag_slot` at every peer (and at this rank itself).
__device__ __forceinline__ void signal_when_grid_done(const Peers& peers, int64_t off_flags, int flag_slot, int W,
                                                      int rank, uint32_t epoch, int32_t* cta_counter) {
  __shared__ int last;
  __threadfence_system();  // this thread's peer stores are ordered before what follows, system-wide
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(cta_counter, 1);
    last = done == (int)gridDim.x - 1;
    if (last) *cta_counter = 0;  // ready for the next launch (stream order separates the launches)
  }
  __syncthreads();
  if (last && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x] + off_flags) + (int64_t)flag_slot * W + rank,
                   epoch);
  }
}

__global__ void __launch_bounds__(kXThreads)
put_kernel(Peers peers, PutArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kXWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kXWarps;
  const int hvecs = (int)(a.hidden_row_bytes >> 4);
  // Rows are taken round-robin over the DESTINATIONS (unit u -> destination (u + rank) % W, its (u / W)-th row), so a
  // rank stores to all of its peers at once and every peer's ingress carries one W-th of every sender's stream at any
  // moment, however far the ranks have drifted apart.  (In plain send order all ranks would store to rank 0 first, then
  // to rank 1, ...: one GPU's ingress at a time carries the whole exchange.)
  int64_t longest = 0;   // rows of the largest destination block
  for (int d = 0; d < a.W; d++) {
    const int jb = d * a.S + (a.stage < 0 ? 0 : a.stage), je = d * a.S + (a.stage < 0 ? a.S - 1 : a.stage);
    const int64_t lo = jb == 0 ? 0 : a.send_incl[jb - 1], hi = a.send_incl[je];
    longest = hi - lo > longest ? hi - lo : longest;
  }
  if (a.T <= 0) longest = 0;
  for (int64_t u = warp; u < longest * a.W; u += n_warps) {
    const int dest_u = (int)((u + a.rank) % a.W);
    const int jb = dest_u * a.S + (a.stage < 0 ? 0 : a.stage), je = dest_u * a.S + (a.stage < 0 ? a.S - 1 : a.stage);
    const int64_t lo = jb == 0 ? 0 : a.send_incl[jb - 1], hi = a.send_incl[je];
    const int64_t i = lo + u / a.W;
    if (i >= hi) continue;
    // window j = (dest, stage) of row i: the first j in [jb, je] with i < send_incl[j]
    int j = jb;
    while (j < je && i >= a.send_incl[j]) j++;
    const int dest = dest_u;
    const int64_t begin = j == 0 ? 0 : a.send_incl[j - 1];
    const int64_t r = (int64_t)a.disp_off[j] + (i - begin);
    const int t = a.send_map[i] % a.T;
    uint8_t* base = peers.base[dest];
    if (a.mask & EPSB_PUT_META) {
      if (lane < a.k) {
        reinterpret_cast<int32_t*>(base + a.off_idx)[r * a.k + lane] = a.idx[(int64_t)t * a.k + lane];
        reinterpret_cast<float*>(base + a.off_wts)[r * a.k + lane] = a.wts[(int64_t)t * a.k + lane];
      }
    }
    if ((a.mask & EPSB_PUT_SCALES) && a.scales != nullptr) {
      float* d = reinterpret_cast<float*>(base + a.off_scales) + r * a.scales_dim;
      for (int c = lane; c < a.scales_dim; c += 32) d[c] = a.scales[(int64_t)t * a.scales_dim + c];
    }
    if (a.mask & EPSB_PUT_HIDDEN)
      copy_row16(a.hidden + (int64_t)t * a.hidden_row_bytes, base + a.off_hidden + r * a.hidden_row_bytes, hvecs, lane);
  }
  signal_when_grid_done(peers, a.off_flags, a.flag_slot, a.W, a.rank, a.epoch, a.cta_counter);
}

__global__ void wait_kernel(const uint8_t* my_base, int64_t off_flags, int flag_slot, int W, uint32_t epoch,
                            uint64_t limit_ns, int code, int32_t* status) {
  if (threadIdx.x < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(my_base + off_flags) + (int64_t)flag_slot * W + threadIdx.x;
    if (!wait_flag(f, epoch, limit_ns) && status != nullptr) {
      atomicCAS(status, 0, code);
      atomicExch(status + 1, (int)threadIdx.x);
    }
  }
}

// ---------------------------------------------------------------- local reduce + put (return trip)

__device__ __forceinline__ void acc8(float (&a)[8], uint4 v) {
  a[0] += bf16_lo(v.x); a[1] += bf16_hi(v.x);
  a[2] += bf16_lo(v.y); a[3] += bf16_hi(v.y);
  a[4] += bf16_lo(v.z); a[5] += bf16_hi(v.z);
  a[6] += bf16_lo(v.w); a[7] += bf16_hi(v.w);
}

// Return row q (block of source rank d, stages [s0, s1)) = bf16(sum_j float(y[red_map[q,j],:])), fp32 accumulation in
// slot order, rows of y already carry their gate weight; stored at row comb_off[d*S+s0] + (q - block begin) of
// rank d's collect arena.
template <int kSlots>
__global__ void __launch_bounds__(kXThreads)
local_reduce_put_kernel(Peers peers, const uint8_t* __restrict__ y, const int32_t* __restrict__ red_map,
                        const int32_t* __restrict__ ret_incl, const int32_t* __restrict__ comb_off, int64_t off_out,
                        int64_t off_flags, int flag_slot, int k, int W, int S, int stage, int64_t H, int rank,
                        uint32_t epoch, int32_t* cta_counter) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kXWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kXWarps;
  const int vecs = (int)(H >> 3);
  const int64_t row_bytes = H * 2;
  const int64_t sentinel = (int64_t)ret_incl[W * S - 1] * k;
  const int s0 = stage < 0 ? 0 : stage, s1 = stage < 0 ? S : stage + 1;
  // rows round-robin over the destinations, like put_kernel: unit u -> destination (u + rank) % W, its (u / W)-th row
  int64_t longest = 0;
  for (int d = 0; d < W; d++) {
    const int jb = d * S + s0, je = d * S + s1 - 1;
    const int64_t b = jb == 0 ? 0 : ret_incl[jb - 1], e = ret_incl[je];
    longest = e - b > longest ? e - b : longest;
  }
  {
    for (int64_t u = warp; u < longest * W; u += n_warps) {   // (the extra brace keeps the loop body's indentation)
      const int d = (int)((u + rank) % W);
      const int jb = d * S + s0, je = d * S + s1 - 1;
      const int64_t b = jb == 0 ? 0 : ret_incl[jb - 1], e = ret_incl[je];
      const int64_t q = b + u / W;
      if (q >= e) continue;
      uint8_t* dst_base = peers.base[d] + off_out + (int64_t)comb_off[jb] * row_bytes;
      int32_t rows[kSlots];
#pragma unroll
      for (int j = 0; j < kSlots; j++) {
        rows[j] = -1;
        if (j < k) {
          const int32_t r = __ldg(red_map + q * k + j);
          if (r < sentinel) rows[j] = r;
        }
      }
      uint8_t* dst = dst_base + (q - b) * row_bytes;
      for (int v = lane; v < vecs; v += 32) {
        uint4 in[kSlots];
#pragma unroll
        for (int j = 0; j < kSlots; j++)
          if (j < k && rows[j] >= 0) in[j] = ld_nc_16(y + (int64_t)rows[j] * row_bytes + (int64_t)v * 16);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < kSlots; j++)
          if (j < k && rows[j] >= 0) acc8(acc, in[j]);
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        st_16(dst + (int64_t)v * 16, o);
      }
    }
  }
  signal_when_grid_done(peers, off_flags, flag_slot, W, rank, epoch, cta_counter);
}

// ---------------------------------------------------------------- fast_oep: ids out, table rows back

// Position pos of the arranged order (ids grouped by owner rank) goes to owner p's id arena.
__global__ void __launch_bounds__(kXThreads)
put_ids_kernel(Peers peers, const int32_t* __restrict__ ids, const int32_t* __restrict__ send_map,
               const int32_t* __restrict__ send_incl, const int32_t* __restrict__ disp_off, int64_t off_idx,
               int64_t off_flags, int flag_slot, int W, int rank, uint32_t epoch, int32_t* cta_counter) {
  const int n_sent = send_incl[W - 1];
  for (int pos = blockIdx.x * kXThreads + threadIdx.x; pos < n_sent; pos += gridDim.x * kXThreads) {
    int p = 0;
    while (p < W - 1 && pos >= send_incl[p]) p++;
    const int begin = p == 0 ? 0 : send_incl[p - 1];
    reinterpret_cast<int32_t*>(peers.base[p] + off_idx)[disp_off[p] + (pos - begin)] = ids[send_map[pos]];
  }
  signal_when_grid_done(peers, off_flags, flag_slot, W, rank, epoch, cta_counter);
}

// The owner side: received id q (from source r) selects a row of this rank's table shard; the row is stored at
// position comb_off[r] + (q - block begin) of r's row arena, i.e. at the id's position in r's arranged order
// (reference lookupKernel + the combine All2All, fast_oep_kernels.cu:186-216, fast_oep.cu:105-133).
__global__ void __launch_bounds__(kXThreads)
lookup_put_kernel(Peers peers, const int32_t* __restrict__ recv_ids, const int32_t* __restrict__ recv_incl,
                  const int32_t* __restrict__ comb_off, const uint8_t* __restrict__ table, int64_t size_per_rank,
                  int64_t row_bytes, int64_t off_out, int64_t off_flags, int flag_slot, int W, int rank, uint32_t epoch,
                  int32_t* cta_counter) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kXWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kXWarps;
  const int vecs = (int)(row_bytes >> 4);
  const int R = recv_incl[W - 1];
  const int first_dest = (rank + 1) % W;   // cyclic from the right-hand neighbour on, like put_kernel
  const int64_t shift = first_dest == 0 ? 0 : recv_incl[first_dest - 1];
  for (int64_t q0 = warp; q0 < R; q0 += n_warps) {
    const int64_t q = q0 + shift < R ? q0 + shift : q0 + shift - R;
    int r = 0;
    while (r < W - 1 && q >= recv_incl[r]) r++;
    const int64_t begin = r == 0 ? 0 : recv_incl[r - 1];
    const int64_t local = (int64_t)recv_ids[q] % size_per_rank;
    copy_row16(table + local * row_bytes, peers.base[r] + off_out + ((int64_t)comb_off[r] + (q - begin)) * row_bytes,
               vecs, lane);
  }
  signal_when_grid_done(peers, off_flags, flag_slot, W, rank, epoch, cta_counter);
}

Peers peers_of(const epsb_exchange* x) {
  Peers p;
  for (int i = 0; i < kMaxPeers; i++) p.base[i] = x->peer[i < x->W ? i : 0];
  return p;
}

int grid_for_rows(int64_t rows) {
  int64_t want = (rows + kXWarps - 1) / kXWarps;
  const int64_t cap = (int64_t)sm_count() * 4;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

constexpr int kDevWords = 16;  // scratch words in front of the offset arrays

}  // namespace

}  // namespace epsb

using namespace epsb;

// ---------------------------------------------------------------- symmetric memory (CUDA IPC)

extern "C" int epsb_symm_alloc(int64_t bytes, void** ptr, uint8_t* handle64) {
  EPSB_REQUIRE(bytes > 0 && ptr != nullptr && handle64 != nullptr, EPSB_ERR_INVALID, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == EPSB_IPC_HANDLE_BYTES, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, (size_t)bytes);  // flags start below every epoch
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(EPSB_ERR_CUDA, "symmetric allocation: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return EPSB_OK;
}

extern "C" int epsb_symm_open(const uint8_t* handle64, void** ptr) {
  EPSB_REQUIRE(handle64 != nullptr && ptr != nullptr, EPSB_ERR_INVALID, "bad arguments");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *ptr = p;
  return EPSB_OK;
}

extern "C" int epsb_symm_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return EPSB_OK;
}

extern "C" int epsb_symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(EPSB_ERR_CUDA, "cudaFree: %s", cudaGetErrorString(e));
  return EPSB_OK;
}

// ---------------------------------------------------------------- exchange object

static int check_shape(int W, int max_tok, int S, int k, int64_t H, int hidden_elem, int scales_dim) {
  EPSB_REQUIRE(W >= 1 && W <= kMaxPeers, EPSB_ERR_INVALID, "ep_world_size %d is outside [1, %d]", W, kMaxPeers);
  EPSB_REQUIRE(max_tok >= 0 && S >= 1 && k >= 1 && k <= 32, EPSB_ERR_INVALID, "bad sizes max_tok=%d S=%d k=%d", max_tok,
               S, k);
  EPSB_REQUIRE((int64_t)W * S <= 1024, EPSB_ERR_INVALID, "ep_world_size * num_stages is too big.");
  EPSB_REQUIRE(H > 0 && H % 8 == 0 && hidden_elem >= 0 && hidden_elem <= 2 && (H * hidden_elem) % 16 == 0,
               EPSB_ERR_INVALID, "hidden size %lld x %d bytes is not a multiple of 16 bytes", (long long)H, hidden_elem);
  EPSB_REQUIRE(scales_dim >= 0, EPSB_ERR_INVALID, "scales_dim %d is negative", scales_dim);
  return EPSB_OK;
}

extern "C" int epsb_exchange_region_bytes(int W, int max_tok, int S_max, int k, int64_t H, int hidden_elem_bytes,
                                          int scales_dim, int64_t* bytes) {
  int rc = check_shape(W, max_tok, S_max, k, H, hidden_elem_bytes, scales_dim);
  if (rc) return rc;
  *bytes = make_layout(max_tok, W, S_max, k, H, hidden_elem_bytes, scales_dim).total;
  return EPSB_OK;
}

extern "C" int epsb_exchange_create(int rank, int W, int max_tok, int S_max, int k, int64_t H, int hidden_elem_bytes,
                                    int scales_dim, void* const* peer_regions, epsb_exchange_t** out) {
  int rc = check_shape(W, max_tok, S_max, k, H, hidden_elem_bytes, scales_dim);
  if (rc) return rc;
  EPSB_REQUIRE(rank >= 0 && rank < W && peer_regions != nullptr && out != nullptr, EPSB_ERR_INVALID, "bad rank %d/%d",
               rank, W);
  epsb_exchange* x = new (std::nothrow) epsb_exchange();
  EPSB_REQUIRE(x != nullptr, EPSB_ERR_INVALID, "out of host memory");
  x->rank = rank; x->W = W; x->max_tok = max_tok; x->S = S_max; x->k = k; x->H = H;
  x->hidden_elem = hidden_elem_bytes; x->scales_dim = scales_dim;
  x->lay = make_layout(max_tok, W, S_max, k, H, hidden_elem_bytes, scales_dim);
  for (int i = 0; i < kMaxPeers; i++) x->peer[i] = nullptr;
  for (int i = 0; i < W; i++) {
    x->peer[i] = static_cast<uint8_t*>(peer_regions[i]);
    if (x->peer[i] == nullptr) {
      delete x;
      return fail(EPSB_ERR_INVALID, "peer region %d is NULL", i);
    }
  }
  const size_t words = kDevWords + 3 * (size_t)W * S_max;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&x->dev), words * 4);
  if (e == cudaSuccess) e = cudaMemset(x->dev, 0, words * 4);
  if (e != cudaSuccess) {
    delete x;
    return fail(EPSB_ERR_CUDA, "exchange scratch: %s", cudaGetErrorString(e));
  }
  x->epoch = 0;
  *out = x;
  return EPSB_OK;
}

extern "C" int epsb_exchange_destroy(epsb_exchange_t* x) {
  if (x == nullptr) return EPSB_OK;
  cudaFree(x->dev);
  delete x;
  return EPSB_OK;
}

extern "C" int epsb_exchange_begin(epsb_exchange_t* x, int* epoch) {
  EPSB_REQUIRE(x != nullptr, EPSB_ERR_INVALID, "exchange handle is NULL");
  x->epoch += 1;
  if (epoch != nullptr) *epoch = x->epoch;
  return EPSB_OK;
}

extern "C" int epsb_exchange_arena(epsb_exchange_t* x, int which, int parity, void** ptr) {
  EPSB_REQUIRE(x != nullptr && ptr != nullptr, EPSB_ERR_INVALID, "bad arguments");
  uint8_t* b = x->peer[x->rank];
  const int par = parity & 1;
  switch (which) {
    case EPSB_ARENA_IDX: *ptr = b + x->lay.idx + par * x->lay.idx_bytes; break;
    case EPSB_ARENA_WEIGHTS: *ptr = b + x->lay.wts + par * x->lay.wts_bytes; break;
    case EPSB_ARENA_HIDDEN: *ptr = b + x->lay.hidden + par * x->lay.hidden_bytes; break;
    case EPSB_ARENA_SCALES: *ptr = b + x->lay.scales + par * x->lay.scales_bytes; break;
    case EPSB_ARENA_OUT: *ptr = b + x->lay.out; break;
    case EPSB_ARENA_RECV_PLAN: *ptr = x->dev + kDevWords + 2 * (int64_t)x->W * x->S; break;
    default: return fail(EPSB_ERR_INVALID, "unknown arena %d", which);
  }
  return EPSB_OK;
}

extern "C" int epsb_exchange_publish_plans(epsb_exchange_t* x, const int32_t* send_incl, const int32_t* coll_incl,
                                           int S, void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(S >= 1 && S <= x->S, EPSB_ERR_INVALID, "Invalid num_stages: %d (exchange was created for %d)", S, x->S);
  publish_plans_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      peers_of(x), x->lay.table_send, x->lay.table_coll, x->lay.flags, x->rank, x->W, x->W * S, x->W * x->S,
      (uint32_t)x->epoch, send_incl, coll_incl);
  return check_launch("exchange_publish_plans");
}

extern "C" int epsb_exchange_recv_plans(epsb_exchange_t* x, int S, int32_t* recv_incl, int32_t* status,
                                        int64_t timeout_ns, void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(S >= 1 && S <= x->S, EPSB_ERR_INVALID, "Invalid num_stages: %d (exchange was created for %d)", S, x->S);
  const int64_t n = (int64_t)x->W * x->S;
  int32_t* off = x->dev + kDevWords;
  recv_plans_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      x->peer[x->rank], x->lay.table_send, x->lay.table_coll, x->lay.flags, x->rank, x->W, S, x->W * x->S,
      (uint32_t)x->epoch, (uint64_t)(timeout_ns > 0 ? timeout_ns : EPSB_EXCHANGE_DEFAULT_TIMEOUT_NS),
      (x->max_tok > 0 ? x->max_tok : 1) * x->W, off + 2 * n, off, off + n, recv_incl, status);
  return check_launch("exchange_recv_plans");
}

extern "C" int epsb_exchange_put(epsb_exchange_t* x, int flag_slot, int stage, int mask, const int32_t* idx,
                                 const float* weights, const void* hidden, const float* scales,
                                 const int32_t* send_map, const int32_t* send_incl, int T, int S, void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(S >= 1 && S <= x->S && stage < S, EPSB_ERR_INVALID, "bad stage %d of %d", stage, S);
  EPSB_REQUIRE(flag_slot >= 1 && flag_slot < 2 + 2 * x->S, EPSB_ERR_INVALID, "bad flag slot %d", flag_slot);
  EPSB_REQUIRE(T >= 0 && T <= x->max_tok, EPSB_ERR_INVALID, "num_tokens %d exceeds max_num_tokens_per_gpu %d", T,
               x->max_tok);
  EPSB_REQUIRE(!(mask & EPSB_PUT_META) || T == 0 || (idx != nullptr && weights != nullptr), EPSB_ERR_INVALID,
               "EPSB_PUT_META needs idx and weights");
  EPSB_REQUIRE(!(mask & EPSB_PUT_HIDDEN) || T == 0 || (hidden != nullptr && ((uintptr_t)hidden & 15) == 0),
               EPSB_ERR_INVALID, "EPSB_PUT_HIDDEN needs a 16-byte aligned hidden buffer");
  EPSB_REQUIRE(!(mask & EPSB_PUT_HIDDEN) || x->hidden_elem > 0, EPSB_ERR_INVALID,
               "this exchange was created without hidden arenas");
  EPSB_REQUIRE(!(mask & EPSB_PUT_SCALES) || T == 0 || x->scales_dim == 0 || scales != nullptr, EPSB_ERR_INVALID,
               "EPSB_PUT_SCALES needs scales");
  const int par = x->epoch & 1;
  const int64_t n = (int64_t)x->W * x->S;
  PutArgs a;
  a.idx = idx; a.wts = weights; a.hidden = static_cast<const uint8_t*>(hidden); a.scales = scales;
  a.send_map = send_map; a.send_incl = send_incl; a.disp_off = x->dev + kDevWords;
  a.off_idx = x->lay.idx + par * x->lay.idx_bytes;
  a.off_wts = x->lay.wts + par * x->lay.wts_bytes;
  a.off_hidden = x->lay.hidden + par * x->lay.hidden_bytes;
  a.off_scales = x->lay.scales + par * x->lay.scales_bytes;
  a.off_flags = x->lay.flags;
  a.hidden_row_bytes = x->H * x->hidden_elem;
  a.T = T; a.k = x->k; a.scales_dim = x->scales_dim; a.W = x->W; a.S = S; a.stage = stage;
  a.mask = x->scales_dim == 0 ? (mask & ~EPSB_PUT_SCALES) : mask;
  a.flag_slot = flag_slot; a.rank = x->rank; a.epoch = (uint32_t)x->epoch;
  a.cta_counter = x->dev + 0;
  (void)n;
  const int64_t rows = (int64_t)T * (x->W < x->k ? x->W : x->k);
  put_kernel<<<grid_for_rows(rows), kXThreads, 0, static_cast<cudaStream_t>(stream)>>>(peers_of(x), a);
  return check_launch("exchange_put");
}

extern "C" int epsb_exchange_wait(epsb_exchange_t* x, int flag_slot, int32_t* status, int64_t timeout_ns,
                                  void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(flag_slot >= 1 && flag_slot < 2 + 2 * x->S, EPSB_ERR_INVALID, "bad flag slot %d", flag_slot);
  wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      x->peer[x->rank], x->lay.flags, flag_slot, x->W, (uint32_t)x->epoch,
      (uint64_t)(timeout_ns > 0 ? timeout_ns : EPSB_EXCHANGE_DEFAULT_TIMEOUT_NS), EPSB_EXCHANGE_TIMEOUT_DATA + flag_slot,
      status);
  return check_launch("exchange_wait");
}

extern "C" int epsb_exchange_local_reduce_put(epsb_exchange_t* x, int flag_slot, const void* y, const int32_t* red_map,
                                              const int32_t* ret_incl, int S, int stage, int64_t max_rows,
                                              void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(S >= 1 && S <= x->S && stage < S, EPSB_ERR_INVALID, "bad stage %d of %d", stage, S);
  EPSB_REQUIRE(flag_slot >= 1 && flag_slot < 2 + 2 * x->S, EPSB_ERR_INVALID, "bad flag slot %d", flag_slot);
  EPSB_REQUIRE(x->k <= 16, EPSB_ERR_INVALID, "top-k %d exceeds 16", x->k);
  const int64_t n = (int64_t)x->W * x->S;
  const int32_t* comb_off = x->dev + kDevWords + n;
  const int grid = grid_for_rows(max_rows > 0 ? max_rows : 1);
  auto st = static_cast<cudaStream_t>(stream);
  if (x->k <= 8)
    local_reduce_put_kernel<8><<<grid, kXThreads, 0, st>>>(peers_of(x), static_cast<const uint8_t*>(y), red_map,
                                                           ret_incl, comb_off, x->lay.out, x->lay.flags, flag_slot,
                                                           x->k, x->W, S, stage, x->H, x->rank, (uint32_t)x->epoch,
                                                           x->dev + 1);
  else
    local_reduce_put_kernel<16><<<grid, kXThreads, 0, st>>>(peers_of(x), static_cast<const uint8_t*>(y), red_map,
                                                            ret_incl, comb_off, x->lay.out, x->lay.flags, flag_slot,
                                                            x->k, x->W, S, stage, x->H, x->rank, (uint32_t)x->epoch,
                                                            x->dev + 1);
  return check_launch("exchange_local_reduce_put");
}

// ---------------------------------------------------------------- fast_oep entry points

extern "C" int epsb_exchange_put_ids(epsb_exchange_t* x, int flag_slot, const int32_t* ids, const int32_t* send_map,
                                     const int32_t* send_incl, int64_t n, void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(flag_slot >= 1 && flag_slot < 2 + 2 * x->S, EPSB_ERR_INVALID, "bad flag slot %d", flag_slot);
  EPSB_REQUIRE(x->k == 1, EPSB_ERR_INVALID, "an id exchange needs an exchange created with k = 1");
  EPSB_REQUIRE(n >= 0 && n <= (int64_t)(x->max_tok > 0 ? x->max_tok : 1) * x->W, EPSB_ERR_INVALID,
               "%lld ids exceed the arena", (long long)n);
  const int par = x->epoch & 1;
  int64_t blocks = (n + kXThreads - 1) / kXThreads;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  if (blocks < 1) blocks = 1;
  put_ids_kernel<<<(int)blocks, kXThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      peers_of(x), ids, send_map, send_incl, x->dev + kDevWords, x->lay.idx + par * x->lay.idx_bytes, x->lay.flags,
      flag_slot, x->W, x->rank, (uint32_t)x->epoch, x->dev + 0);
  return check_launch("exchange_put_ids");
}

extern "C" int epsb_exchange_lookup_put(epsb_exchange_t* x, int flag_slot, const void* table, int64_t size_per_rank,
                                        int64_t max_rows, void* stream) {
  EPSB_REQUIRE(x != nullptr && x->epoch > 0, EPSB_ERR_INVALID, "call epsb_exchange_begin first");
  EPSB_REQUIRE(flag_slot >= 1 && flag_slot < 2 + 2 * x->S, EPSB_ERR_INVALID, "bad flag slot %d", flag_slot);
  EPSB_REQUIRE(x->k == 1 && size_per_rank > 0 && table != nullptr && ((uintptr_t)table & 15) == 0, EPSB_ERR_INVALID,
               "bad table / size_per_rank");
  const int par = x->epoch & 1;
  const int64_t n = (int64_t)x->W * x->S;
  const int32_t* recv_ids = reinterpret_cast<const int32_t*>(x->peer[x->rank] + x->lay.idx + par * x->lay.idx_bytes);
  lookup_put_kernel<<<grid_for_rows(max_rows > 0 ? max_rows : 1), kXThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      peers_of(x), recv_ids, x->dev + kDevWords + 2 * n, x->dev + kDevWords + n, static_cast<const uint8_t*>(table),
      size_per_rank, x->H * 2, x->lay.out, x->lay.flags, flag_slot, x->W, x->rank, (uint32_t)x->epoch, x->dev + 1);
  return check_launch("exchange_lookup_put");
}
