// The cached side of a latent attention: a token's compressed key/value vector.
//
// A layer with a down-projection of its own turns each token's projection (rank numbers) into
// c = x / sqrt(mean(x^2) + eps) * gain and keeps only c, in a paged cache with one "head" of
// size rank and no separate values.  Keys and values of every head are linear maps of c, so the
// attention itself runs on c: the queries are first carried through the key map
// (q'_h = Wuk_h^T q_h, so that q_h . k_h = q'_h . c), the attention is then a multi-query one whose
// keys and values are both c, and its result is carried through the value map afterwards.  This
// file holds the norm-and-store step; the two per-head maps are batched products (gemm_simt.cu)
// and the attention is the paged multi-query kernels that the other mixers use.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

// One warp per token: sum of squares, reciprocal root and scaling in float32; the result is
// rounded to the cache's element type once and written at the token's place in the pages.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_norm_store_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ gain, float eps,
                         const int* __restrict__ slot_map, T* __restrict__ pages, int n_tokens, int rank, int row_width) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= n_tokens) return;
  const T* row = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float v = to_f32(row[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)rank + eps);
  T* dst = pages + (size_t)slot_map[t] * row_width;
  for (int c = lane; c < rank; c += 32) dst[c] = from_f32<T>(to_f32(row[c]) * r * gain[c]);
  for (int c = rank + lane; c < row_width; c += 32) dst[c] = from_f32<T>(0.f);      // a row wider than the rank ends in zeros
}

}  // namespace

// x [n_tokens, x_stride]: the first `rank` columns of a row are the token's projection.
// pages [pages, 1, page_size, row_width] with row_width >= rank (a cache whose rows are padded to a width
// that the attention kernels take; the padding is written as zeros); slot_map[t] = page * page_size + offset.
LLMK_API int llmk_latent_norm_store(const void* x, long long x_stride, const float* gain, float eps,
                                    const int* slot_map, void* pages, int n_tokens, int rank, int row_width, int dtype,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  LLMK_REQUIRE(rank > 0 && x_stride >= rank && row_width >= rank, "latent_norm_store: bad rank %d, width %d or stride %lld", rank, row_width, x_stride);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = LLMK_ELEM(tag);
    launch_kernel(latent_norm_store_kernel<T>, dim3((n_tokens + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream,
                  (const T*)x, x_stride, gain, eps, slot_map, (T*)pages, n_tokens, rank, row_width);
    LLMK_LAUNCH_CHECK("latent_norm_store");
  });
}
