// TP <-> DP conversion of [tokens, hidden] bf16 rows inside a tensor-parallel group of one NVSwitch box.
//
// Replaces the reference's TPDPConvertor (src/communication/tp_dp_convertor.cu:54-129) and its runners
// (src/communication/allgather_runner.cu:13-83, reducescatter_runner.cu:61-122): every rank of the group owns one
// symmetric buffer of buffer_rows rows (the reference sizes it attn_tp_size * tp_max_num_tokens rows,
// tp_dp_convertor.cuh:17-19); a call works on tp_num_tokens rows, of which rank r owns the slice
// [offset_r, offset_r + n_r) with n_r = tp_num_tokens / tp_size (+1 for the first tp_num_tokens % tp_size ranks),
// exactly the reference's split (tp_dp_convertor.cu:54-62).
//   all-gather      every rank stores its slice into every peer's buffer (peer stores);
//   reduce-scatter  every rank reads its slice from every peer's buffer (peer loads), sums in fp32 in rank order and
//                   writes the bf16 result over its own slice.
// Synchronisation is by flag words in the regions (epoch valued, never reset): "ready" before anybody touches a
// peer's buffer, "done" before anybody reuses its own.  Signal, wait and data movement are separate launches so
// that every spin is a bounded wait on flags other launches set; after its limit a wait records a code in the
// caller's status words and returns.
#include "common.cuh"

namespace epsb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 4;

struct Group {
  uint8_t* base[EPSB_MAX_PEERS];
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

__device__ __forceinline__ void slice_of(int r, int tp_size, int64_t tokens, int64_t& off, int64_t& n) {
  const int64_t q = tokens / tp_size, rem = tokens % tp_size;
  n = q + (r < rem ? 1 : 0);
  off = q * r + (r < rem ? r : rem);
}

__global__ void signal_kernel(Group g, int64_t flags_off, int slot, int tp_rank, int tp_size, uint32_t epoch) {
  if ((int)threadIdx.x < tp_size) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(g.base[threadIdx.x] + flags_off) + slot * EPSB_MAX_PEERS + tp_rank, epoch);
  }
}

__global__ void wait_kernel(const uint8_t* mine, int64_t flags_off, int slot, int tp_size, uint32_t epoch,
                            uint64_t limit_ns, int32_t* status) {
  if ((int)threadIdx.x >= tp_size) return;
  const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + flags_off) + slot * EPSB_MAX_PEERS + threadIdx.x;
  const uint64_t t0 = now_ns();
  while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
    if (now_ns() - t0 > limit_ns) {
      if (status != nullptr) {
        atomicCAS(status, 0, EPSB_TPDP_TIMEOUT + slot);
        atomicExch(status + 1, (int)threadIdx.x);
      }
      return;
    }
    __nanosleep(64);
  }
}

__device__ __forceinline__ void signal_when_grid_done(const Group& g, int64_t flags_off, int slot, int tp_rank,
                                                      int tp_size, uint32_t epoch, int32_t* counter) {
  __shared__ int last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    last = atomicAdd(counter, 1) == (int)gridDim.x - 1;
    if (last) *counter = 0;
  }
  __syncthreads();
  if (last && (int)threadIdx.x < tp_size) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(g.base[threadIdx.x] + flags_off) + slot * EPSB_MAX_PEERS + tp_rank, epoch);
  }
}

__global__ void __launch_bounds__(kThreads)
all_gather_put_kernel(Group g, int64_t flags_off, int slot, int tp_rank, int tp_size, int64_t tokens,
                      int64_t row_bytes, uint32_t epoch, int32_t* counter) {
  int64_t off, n;
  slice_of(tp_rank, tp_size, tokens, off, n);
  const int64_t vecs = n * row_bytes / 16;   // the slice is contiguous
  const uint4* src = reinterpret_cast<const uint4*>(g.base[tp_rank] + off * row_bytes);
  for (int p = 0; p < tp_size; p++) {
    if (p == tp_rank) continue;
    uint4* dst = reinterpret_cast<uint4*>(g.base[p] + off * row_bytes);
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < vecs; v += (int64_t)gridDim.x * kThreads)
      st_16(dst + v, ld_nc_16(src + v));
  }
  signal_when_grid_done(g, flags_off, slot, tp_rank, tp_size, epoch, counter);
}

__global__ void __launch_bounds__(kThreads)
reduce_scatter_sum_kernel(Group g, int64_t flags_off, int slot, int tp_rank, int tp_size, int64_t tokens,
                          int64_t row_bytes, uint32_t epoch, int32_t* counter) {
  int64_t off, n;
  slice_of(tp_rank, tp_size, tokens, off, n);
  const int64_t vecs = n * row_bytes / 16;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < vecs; v += (int64_t)gridDim.x * kThreads) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < tp_size; p++) {   // rank order: every rank of the group would compute the same bits
      const uint4 x = ld_nc_16(reinterpret_cast<const uint4*>(g.base[p] + off * row_bytes) + v);
      a[0] += bf16_lo(x.x); a[1] += bf16_hi(x.x);
      a[2] += bf16_lo(x.y); a[3] += bf16_hi(x.y);
      a[4] += bf16_lo(x.z); a[5] += bf16_hi(x.z);
      a[6] += bf16_lo(x.w); a[7] += bf16_hi(x.w);
    }
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]);
    o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]);
    o.w = pack_bf16x2(a[6], a[7]);
    st_16(reinterpret_cast<uint4*>(g.base[tp_rank] + off * row_bytes) + v, o);
  }
  signal_when_grid_done(g, flags_off, slot, tp_rank, tp_size, epoch, counter);
}

int64_t data_bytes(int64_t buffer_rows, int64_t hidden) {
  return ((buffer_rows > 0 ? buffer_rows : 1) * hidden * 2 + 255) & ~(int64_t)255;
}

int fill_group(Group& g, void* const* regions, int tp_size) {
  EPSB_REQUIRE(regions != nullptr && tp_size >= 1 && tp_size <= EPSB_MAX_PEERS, EPSB_ERR_INVALID,
               "attn_tp_size %d is outside [1, %d]", tp_size, EPSB_MAX_PEERS);
  for (int i = 0; i < EPSB_MAX_PEERS; i++) g.base[i] = static_cast<uint8_t*>(regions[i < tp_size ? i : 0]);
  return EPSB_OK;
}

int grid_for(int64_t bytes) {
  int64_t want = (bytes / 16 + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 4;
  if (want > cap) want = cap;
  return (int)(want < 1 ? 1 : want);
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_tpdp_region_bytes(int64_t buffer_rows, int64_t hidden, int64_t* bytes) {
  EPSB_REQUIRE(hidden > 0 && hidden % 8 == 0, EPSB_ERR_INVALID, "hidden size %lld is not a multiple of 8", (long long)hidden);
  *bytes = data_bytes(buffer_rows, hidden) + 256 /* flags */ + 256 /* CTA counter */;
  return EPSB_OK;
}

extern "C" int epsb_tpdp_signal(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows,
                                int64_t hidden, int slot, int epoch, void* stream) {
  Group g;
  int rc = fill_group(g, regions, tp_size);
  if (rc) return rc;
  EPSB_REQUIRE(slot >= 0 && slot < kSlots && tp_rank >= 0 && tp_rank < tp_size, EPSB_ERR_INVALID, "bad slot / rank");
  signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(g, data_bytes(buffer_rows, hidden), slot, tp_rank,
                                                                 tp_size, (uint32_t)epoch);
  return check_launch("tpdp_signal");
}

extern "C" int epsb_tpdp_wait(const void* my_region, int tp_size, int64_t buffer_rows, int64_t hidden, int slot,
                              int epoch, int32_t* status, int64_t timeout_ns, void* stream) {
  EPSB_REQUIRE(my_region != nullptr && slot >= 0 && slot < kSlots && tp_size >= 1 && tp_size <= EPSB_MAX_PEERS,
               EPSB_ERR_INVALID, "bad arguments");
  wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(my_region), data_bytes(buffer_rows, hidden), slot, tp_size, (uint32_t)epoch,
      (uint64_t)(timeout_ns > 0 ? timeout_ns : EPSB_EXCHANGE_DEFAULT_TIMEOUT_NS), status);
  return check_launch("tpdp_wait");
}

static int tpdp_move(bool gather, void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows,
                     int64_t tp_num_tokens, int64_t hidden, int64_t buffer_hidden, int slot, int epoch, void* stream) {
  Group g;
  int rc = fill_group(g, regions, tp_size);
  if (rc) return rc;
  EPSB_REQUIRE(slot >= 0 && slot < kSlots && tp_rank >= 0 && tp_rank < tp_size, EPSB_ERR_INVALID, "bad slot / rank");
  EPSB_REQUIRE(hidden > 0 && hidden % 8 == 0 && hidden <= buffer_hidden, EPSB_ERR_INVALID,
               "%lld should be smaller than or equal to%lld", (long long)hidden, (long long)buffer_hidden);
  EPSB_REQUIRE(tp_num_tokens >= 0 && tp_num_tokens * hidden <= (buffer_rows > 0 ? buffer_rows : 1) * buffer_hidden,
               EPSB_ERR_INVALID, "tp_num_tokens %lld exceeds the buffer", (long long)tp_num_tokens);
  const int64_t flags_off = data_bytes(buffer_rows, buffer_hidden);
  int32_t* counter = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(regions[tp_rank]) + flags_off + 256);
  const int64_t slice_bytes = (tp_num_tokens / tp_size + 1) * hidden * 2;
  auto st = static_cast<cudaStream_t>(stream);
  if (gather)
    all_gather_put_kernel<<<grid_for(slice_bytes), kThreads, 0, st>>>(g, flags_off, slot, tp_rank, tp_size, tp_num_tokens,
                                                                      hidden * 2, (uint32_t)epoch, counter);
  else
    reduce_scatter_sum_kernel<<<grid_for(slice_bytes), kThreads, 0, st>>>(g, flags_off, slot, tp_rank, tp_size,
                                                                          tp_num_tokens, hidden * 2, (uint32_t)epoch,
                                                                          counter);
  return check_launch(gather ? "tpdp_all_gather_put" : "tpdp_reduce_scatter_sum");
}

extern "C" int epsb_tpdp_all_gather_put(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows,
                                        int64_t tp_num_tokens, int64_t hidden, int64_t buffer_hidden, int slot, int epoch,
                                        void* stream) {
  return tpdp_move(true, regions, tp_rank, tp_size, buffer_rows, tp_num_tokens, hidden, buffer_hidden, slot, epoch,
                   stream);
}

extern "C" int epsb_tpdp_reduce_scatter_sum(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows,
                                            int64_t tp_num_tokens, int64_t hidden, int64_t buffer_hidden, int slot,
                                            int epoch, void* stream) {
  return tpdp_move(false, regions, tp_rank, tp_size, buffer_rows, tp_num_tokens, hidden, buffer_hidden, slot, epoch,
                   stream);
}
