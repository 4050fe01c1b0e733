// The cached side of attention over a low-rank vector per token: c = norm(x W_down^T) * w is all that a token leaves
// in the cache; keys and values are linear in c, so the attention itself can run on c (the key expansion moved into
// the query, the value expansion applied to the attention's output).
//
// latent_norm_cache_write_kernel: RMS norm of the projected rows (float32 inside) fused with the write into the
// pages: [page][1][1][slot][padded rank], the padding (rank rounded up to what the attention kernels take) is zero.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_latent_cache)

namespace lmsf {

template <typename T>
__global__ void __launch_bounds__(128) latent_norm_cache_write_kernel(const T* __restrict__ x, long long x_stride,
                                                                      const float* __restrict__ w, T* __restrict__ cache,
                                                                      long long page_stride, const int* __restrict__ positions,
                                                                      const int* __restrict__ token_seq,
                                                                      const int* __restrict__ block_table, int max_blocks,
                                                                      int block_size, int rank, int padded, float eps,
                                                                      int* __restrict__ error_flag) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(xr[i]); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int blk = pos / block_size;
  const int page = blk < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + blk] : -1;
  if (page < 0) {   // no page for this position: a fault of the caller, reported and not written
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  T* dst = cache + (size_t)page * page_stride + (size_t)(pos % block_size) * padded;
  for (int i = threadIdx.x; i < padded; i += blockDim.x)
    dst[i] = i < rank ? from_f32<T>((to_f32(xr[i]) * inv) * w[i]) : from_f32<T>(0.f);
}

// x[t, h, :] *= sigmoid(gate[t, h]): a gate per token and head on the attention's output.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                 int heads, int head_dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * head_dim; i += blockDim.x) {
    const float g = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + i / head_dim])));
    T* p = x + (size_t)t * x_stride + i;
    *p = from_f32<T>(to_f32(*p) * g);
  }
}

}  // namespace lmsf

LMSF_API int lmsf_head_gate(void* x, long long x_stride, const void* gate, long long gate_stride, int n, int heads,
                            int head_dim, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (heads <= 0 || head_dim <= 0) LMSF_REFUSE("head_gate: heads=%d head_dim=%d", heads, head_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) head_gate_kernel<float><<<n, 256, 0, s>>>((float*)x, x_stride, (const float*)gate, gate_stride, heads, head_dim);
  else if (dtype == LMSF_BF16) head_gate_kernel<bf16><<<n, 256, 0, s>>>((bf16*)x, x_stride, (const bf16*)gate, gate_stride, heads, head_dim);
  else LMSF_REFUSE("head_gate: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// x: rows of [n, rank] of `dtype` (row stride x_stride); w: float32 [rank]; cache: [pages, 1, 1, block_size, padded].
LMSF_API int lmsf_latent_norm_cache_write(const void* x, long long x_stride, const float* w, void* cache,
                                          long long page_stride, const int* positions, const int* token_seq,
                                          const int* block_table, int max_blocks, int block_size, int n, int rank, int padded,
                                          float eps, int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (rank <= 0 || padded < rank || block_size <= 0 || max_blocks <= 0 || !(eps > 0.f))
    LMSF_REFUSE("latent cache: rank=%d padded=%d block_size=%d max_blocks=%d", rank, padded, block_size, max_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32)
    latent_norm_cache_write_kernel<float><<<n, 128, 0, s>>>((const float*)x, x_stride, w, (float*)cache, page_stride, positions,
                                                            token_seq, block_table, max_blocks, block_size, rank, padded, eps, error_flag);
  else if (dtype == LMSF_BF16)
    latent_norm_cache_write_kernel<bf16><<<n, 128, 0, s>>>((const bf16*)x, x_stride, w, (bf16*)cache, page_stride, positions,
                                                           token_seq, block_table, max_blocks, block_size, rank, padded, eps, error_flag);
  else LMSF_REFUSE("latent cache: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}
