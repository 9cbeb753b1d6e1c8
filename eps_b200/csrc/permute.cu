// Row gathers / scatters / segment copies of the dispatch and combine paths (sm_100a).
//
// All of them move whole rows of row_bytes (a multiple of 16) with 16-byte
// accesses; a warp owns a row at a time and keeps four vectors per lane in
// flight, and the grid is sized to fill every SM with resident warps, so the
// kernels are bound by HBM rather than by latency.
#include "common.cuh"

namespace epsb {

namespace {

constexpr int kMoveThreads = 256;
constexpr int kMoveWarps = kMoveThreads / 32;

__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int vecs, int lane) {
  int v = lane;
  for (; v + 96 < vecs; v += 128) {
    const uint4 a = ld_nc_16(src + v), b = ld_nc_16(src + v + 32), c = ld_nc_16(src + v + 64),
                d = ld_nc_16(src + v + 96);
    st_16(dst + v, a);
    st_16(dst + v + 32, b);
    st_16(dst + v + 64, c);
    st_16(dst + v + 96, d);
  }
  for (; v < vecs; v += 32) st_16(dst + v, ld_nc_16(src + v));
}

__global__ void __launch_bounds__(kMoveThreads)
gather_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int32_t* __restrict__ map,
                   int32_t map_div, int32_t map_mod, const int32_t* __restrict__ bounds, int b0, int b1,
                   int64_t n_rows, int64_t row_bytes) {
  int64_t begin = 0, end = n_rows;
  if (bounds != nullptr) {
    begin = bounds[b0];
    end = bounds[b1];
  }
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kMoveWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kMoveWarps;
  const int vecs = (int)(row_bytes >> 4);
  for (int64_t i = begin + warp; i < end; i += n_warps) {
    const int32_t m = __ldg(map + i);
    const int64_t s = (int64_t)((m / map_div) % map_mod);
    copy_row(reinterpret_cast<const uint4*>(src + s * row_bytes), reinterpret_cast<uint4*>(dst + i * row_bytes), vecs,
             lane);
  }
}

// Rows that are not a multiple of 16 bytes (index / weight rows of k int32 or fp32): one 4-byte word per thread.
__global__ void __launch_bounds__(kMoveThreads)
gather_words_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, const int32_t* __restrict__ map,
                    int32_t map_div, int32_t map_mod, const int32_t* __restrict__ bounds, int b0, int b1,
                    int64_t n_rows, int words) {
  int64_t begin = 0, end = n_rows;
  if (bounds != nullptr) {
    begin = bounds[b0];
    end = bounds[b1];
  }
  const int64_t total = (end - begin) * words;
  for (int64_t g = (int64_t)blockIdx.x * kMoveThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kMoveThreads) {
    const int64_t i = begin + g / words;
    const int c = (int)(g % words);
    const int32_t m = __ldg(map + i);
    const int64_t s = (int64_t)((m / map_div) % map_mod);
    dst[i * words + c] = __ldg(src + s * words + c);
  }
}

__global__ void __launch_bounds__(kMoveThreads)
scatter_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int32_t* __restrict__ map,
                    int32_t div, int64_t n, int64_t row_bytes) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kMoveWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kMoveWarps;
  const int vecs = (int)(row_bytes >> 4);
  for (int64_t i = warp; i < n; i += n_warps) {
    const int32_t m = __ldg(map + i);
    if (m >= kZcMark) continue;
    copy_row(reinterpret_cast<const uint4*>(src + (i / div) * row_bytes),
             reinterpret_cast<uint4*>(dst + (int64_t)m * row_bytes), vecs, lane);
  }
}

// Segments are handed to CTAs round-robin in chunks of rows so that one long
// segment does not serialise on a single CTA.
__global__ void __launch_bounds__(kMoveThreads)
arrange_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const int32_t* __restrict__ src_off,
                    const int32_t* __restrict__ rows, const int32_t* __restrict__ dst_off, int n_seg,
                    int64_t row_bytes) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kMoveWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kMoveWarps;
  const int vecs = (int)(row_bytes >> 4);
  // Every warp walks the segment list; row r of the concatenation goes to warp r % n_warps.
  int64_t seen = 0;
  for (int p = 0; p < n_seg; p++) {
    const int64_t nr = __ldg(rows + p);
    const int64_t so = __ldg(src_off + p), d_o = __ldg(dst_off + p);
    int64_t first = (warp - seen % n_warps + n_warps) % n_warps;
    for (int64_t i = first; i < nr; i += n_warps)
      copy_row(reinterpret_cast<const uint4*>(src + (so + i) * row_bytes),
               reinterpret_cast<uint4*>(dst + (d_o + i) * row_bytes), vecs, lane);
    seen += nr;
  }
}

__global__ void __launch_bounds__(256)
gather_row_weights_kernel(const float* __restrict__ w_recv, const int32_t* __restrict__ gemm_map,
                          const int32_t* __restrict__ excl, int num_experts, float* __restrict__ row_w) {
  const int64_t D = excl[num_experts];
  for (int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; d < D; d += (int64_t)gridDim.x * blockDim.x)
    row_w[d] = w_recv[gemm_map[d]];
}

// out[dst(i), :] = rows[mapping[i], :] for mapping[i] >= 0; dst(i) = i, or with do_permute the n-gram-major position
// i / n_grams + (i % n_grams) * (n / n_grams) (reference scatterKernel, fast_oep_kernels.cu:218-245).
__global__ void __launch_bounds__(kMoveThreads)
oep_scatter_kernel(const uint8_t* __restrict__ rows, const int32_t* __restrict__ mapping, int64_t n, int64_t row_bytes,
                   int64_t n_grams, int do_permute, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kMoveWarps + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * kMoveWarps;
  const int vecs = (int)(row_bytes >> 4);
  const int64_t batch = n / n_grams;
  for (int64_t i = warp; i < n; i += n_warps) {
    const int32_t m = __ldg(mapping + i);
    if (m < 0) continue;
    const int64_t d = do_permute ? i / n_grams + (i % n_grams) * batch : i;
    copy_row(reinterpret_cast<const uint4*>(rows + (int64_t)m * row_bytes), reinterpret_cast<uint4*>(out + d * row_bytes),
             vecs, lane);
  }
}

// Per GEMM row d < excl[EL]: where its input row comes from and what it is worth.  gemm_map[d] = received row * k +
// slot.  a_rows[d] = the received row, or, when send_map is given (a world of one, where the receive order is the send
// order), the token behind it: send_map[row] % T.  row_w[d] = w_src[a_rows[d] * k + slot].
__global__ void __launch_bounds__(256)
gemm_row_sources_kernel(const int32_t* __restrict__ gemm_map, const int32_t* __restrict__ excl, int num_experts, int k,
                        const int32_t* __restrict__ send_map, int T, const float* __restrict__ w_src,
                        int32_t* __restrict__ a_rows, float* __restrict__ row_w) {
  const int64_t D = excl[num_experts];
  for (int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; d < D; d += (int64_t)gridDim.x * blockDim.x) {
    const int32_t m = gemm_map[d];
    int32_t row = m / k;
    const int slot = m - row * k;
    if (send_map != nullptr) row = send_map[row] % T;
    a_rows[d] = row;
    if (row_w != nullptr) row_w[d] = w_src[(int64_t)row * k + slot];
  }
}

int move_grid(int64_t rows) {
  int64_t want = (rows + kMoveWarps - 1) / kMoveWarps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

int check_rows(const void* a, const void* b, int64_t row_bytes) {
  EPSB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, EPSB_ERR_INVALID, "row_bytes %lld is not a multiple of 16",
               (long long)row_bytes);
  EPSB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0, EPSB_ERR_INVALID,
               "row buffers must be 16-byte aligned");
  return EPSB_OK;
}

}  // namespace

}  // namespace epsb

using namespace epsb;

extern "C" int epsb_gather_rows(const void* src, void* dst, const int32_t* map, int32_t map_div, int32_t map_mod,
                                const int32_t* bounds, int b0, int b1, int64_t n_rows, int64_t max_rows,
                                int64_t row_bytes, void* stream) {
  EPSB_REQUIRE(map_div > 0 && map_mod > 0, EPSB_ERR_INVALID, "map_div/map_mod must be positive");
  const int64_t bound = bounds ? max_rows : n_rows;
  if (row_bytes > 0 && row_bytes % 16 != 0) {
    EPSB_REQUIRE(row_bytes % 4 == 0 && ((uintptr_t)src & 3) == 0 && ((uintptr_t)dst & 3) == 0, EPSB_ERR_INVALID,
                 "row_bytes %lld is not a multiple of 4", (long long)row_bytes);
    if (bound <= 0) return EPSB_OK;
    const int words = (int)(row_bytes / 4);
    int64_t blocks = (bound * words + kMoveThreads - 1) / kMoveThreads;
    if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
    gather_words_kernel<<<(int)blocks, kMoveThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        (const uint32_t*)src, (uint32_t*)dst, map, map_div, map_mod, bounds, b0, b1, n_rows, words);
    return check_launch("gather_rows(words)");
  }
  int rc = check_rows(src, dst, row_bytes);
  if (rc) return rc;
  if (bound <= 0) return EPSB_OK;
  gather_rows_kernel<<<move_grid(bound), kMoveThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)src, (uint8_t*)dst, map, map_div, map_mod, bounds, b0, b1, n_rows, row_bytes);
  return check_launch("gather_rows");
}

extern "C" int epsb_scatter_rows(const void* src, void* dst, const int32_t* map, int32_t div, int64_t n,
                                 int64_t row_bytes, void* stream) {
  int rc = check_rows(src, dst, row_bytes);
  if (rc) return rc;
  EPSB_REQUIRE(div > 0, EPSB_ERR_INVALID, "div must be positive");
  if (n <= 0) return EPSB_OK;
  scatter_rows_kernel<<<move_grid(n), kMoveThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)src, (uint8_t*)dst, map, div, n, row_bytes);
  return check_launch("scatter_rows");
}

extern "C" int epsb_oep_scatter(const void* rows, const int32_t* mapping, int64_t n, int64_t row_bytes, int64_t n_grams,
                                int do_permute, void* out, void* stream) {
  int rc = check_rows(rows, out, row_bytes);
  if (rc) return rc;
  EPSB_REQUIRE(n_grams > 0 && (!do_permute || n % n_grams == 0), EPSB_ERR_INVALID,
               "n_grams %lld does not divide %lld ids", (long long)n_grams, (long long)n);
  if (n <= 0) return EPSB_OK;
  oep_scatter_kernel<<<move_grid(n), kMoveThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)rows, mapping, n, row_bytes, n_grams, do_permute, (uint8_t*)out);
  return check_launch("oep_scatter");
}

extern "C" int epsb_arrange_rows(const void* src, void* dst, const int32_t* src_off, const int32_t* rows,
                                 const int32_t* dst_off, int n_seg, int64_t max_rows, int64_t row_bytes,
                                 void* stream) {
  int rc = check_rows(src, dst, row_bytes);
  if (rc) return rc;
  if (n_seg <= 0 || max_rows <= 0) return EPSB_OK;
  arrange_rows_kernel<<<move_grid(max_rows), kMoveThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)src, (uint8_t*)dst, src_off, rows, dst_off, n_seg, row_bytes);
  return check_launch("arrange_rows");
}

extern "C" int epsb_gemm_row_sources(const int32_t* gemm_map, const int32_t* excl, int num_experts, int k,
                                     const int32_t* send_map, int T, const float* w_src, int64_t max_rows,
                                     int32_t* a_rows, float* row_w, void* stream) {
  EPSB_REQUIRE(k > 0 && num_experts > 0 && (send_map == nullptr || T > 0) && a_rows != nullptr, EPSB_ERR_INVALID,
               "bad arguments k=%d num_experts=%d T=%d", k, num_experts, T);
  EPSB_REQUIRE(row_w == nullptr || w_src != nullptr, EPSB_ERR_INVALID, "row_w needs w_src");
  if (max_rows <= 0) return EPSB_OK;
  int64_t blocks = (max_rows + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  gemm_row_sources_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(gemm_map, excl, num_experts, k,
                                                                                      send_map, T, w_src, a_rows, row_w);
  return check_launch("gemm_row_sources");
}

extern "C" int epsb_gather_row_weights(const float* w_recv, const int32_t* gemm_map, const int32_t* excl,
                                       int num_experts, int64_t max_rows, float* row_w, void* stream) {
  if (max_rows <= 0) return EPSB_OK;
  int64_t blocks = (max_rows + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  gather_row_weights_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(w_recv, gemm_map, excl,
                                                                                        num_experts, row_w);
  return check_launch("gather_row_weights");
}
