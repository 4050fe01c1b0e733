// Linear attention with a decay per head ("lightning attention") and the gated norm that follows it.
//
//   S_t = a_h S_(t-1) + k_t v_t^T      (S: [dk, dv] per request and head, float32, kept across steps in a state slot)
//   o_t = S_t^T q_t
//
// q, k, v arrive as the rows of a projection's output and pass through an activation on the way in (SiLU or none),
// computed in float32 from the stored value; the state, the decay and the output are float32 throughout.
//
// lightning_scan_kernel: one block per (request, head, 32 value columns).  Warp w holds rows [w R, (w + 1) R) of the
// state's 32 columns in registers (one column per lane); the request's tokens are taken in chunks of kChunk whose
// q and k rows are staged in shared memory; every warp walks the chunk token by token and leaves its partial
// outputs in shared memory, which are added up in a fixed order after the chunk.  A request that brings one token
// (a decode step) runs the same code with one chunk of one token: the state is read and written once.
// Any cut of a sequence into steps performs the same operations on the state in the same order, so the results
// do not depend on the cut by a bit.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_lightning)

namespace lmsf {

constexpr int kWarps = 4;
constexpr int kChunk = 16;
constexpr int kMaxDk = 256;

__device__ __forceinline__ float act_in(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }

struct ScanArgs {
  const void* q; const void* k; const void* v;     // rows of [n_tokens, *]; head h starts at h * dk (q, k) or h * dv (v)
  long long q_stride, k_stride, v_stride;
  float* out; long long out_stride;                // [n_tokens, heads * dv] float32
  float* state;                                    // [slots, heads, dk, dv] float32
  const float* decay;                              // [heads]
  const int* cu_q; const int* state_slot;          // [n_seqs + 1], [n_seqs]
  int heads, dk, dv, act;
};

template <typename T, int R>
__global__ void __launch_bounds__(kWarps * 32) lightning_scan_kernel(ScanArgs a) {
  __shared__ float qs[kChunk][kMaxDk];
  __shared__ float ks[kChunk][kMaxDk];
  __shared__ float part[kWarps][kChunk][32];
  const int seq = blockIdx.x, head = blockIdx.y, col = blockIdx.z * 32 + (threadIdx.x & 31);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = a.cu_q[seq], t1 = a.cu_q[seq + 1];
  if (t1 <= t0) return;
  const int dk = a.dk, dv = a.dv;
  const bool live = col < dv;
  const float decay = a.decay[head];
  float* st = a.state + (((size_t)a.state_slot[seq] * a.heads + head) * dk) * dv;
  const int r0 = warp * R;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (live && r0 + i < dk) ? st[(size_t)(r0 + i) * dv + col] : 0.f;

  for (int c0 = t0; c0 < t1; c0 += kChunk) {
    const int n = min(kChunk, t1 - c0);
    __syncthreads();   // the chunk before has been read
    for (int e = threadIdx.x; e < n * dk; e += kWarps * 32) {
      const int t = e / dk, d = e - t * dk;
      qs[t][d] = act_in(to_f32(((const T*)a.q)[(size_t)(c0 + t) * a.q_stride + (size_t)head * dk + d]), a.act);
      ks[t][d] = act_in(to_f32(((const T*)a.k)[(size_t)(c0 + t) * a.k_stride + (size_t)head * dk + d]), a.act);
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float vv = live ? act_in(to_f32(((const T*)a.v)[(size_t)(c0 + t) * a.v_stride + (size_t)head * dv + col]), a.act) : 0.f;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        if (r0 + i < dk) {
          S[i] = fmaf(decay, S[i], ks[t][r0 + i] * vv);
          o = fmaf(qs[t][r0 + i], S[i], o);
        }
      }
      part[warp][t][lane] = o;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * 32; e += kWarps * 32) {
      const int t = e >> 5, l = e & 31;
      const int c = blockIdx.z * 32 + l;
      if (c < dv) {
        float o = part[0][t][l];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) o += part[w][t][l];
        a.out[(size_t)(c0 + t) * a.out_stride + (size_t)head * dv + c] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i)
    if (live && r0 + i < dk) st[(size_t)(r0 + i) * dv + col] = S[i];
}

// out[t] = norm(x[t]) * w * sigmoid(gate[t]) : the norm over all heads of a token together, float32 inside.
// x: float32 [n, width]; gate: rows of the activation type; out: activation type [n, width].  One block per token.
template <typename T>
__global__ void __launch_bounds__(256) gated_norm_kernel(T* __restrict__ out, const float* __restrict__ x, long long x_stride,
                                                         const T* __restrict__ gate, long long gate_stride,
                                                         const float* __restrict__ w, int width, float eps) {
  __shared__ float scratch[33];
  const float* xr = x + (size_t)blockIdx.x * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float g = to_f32(gate[(size_t)blockIdx.x * gate_stride + i]);
    out[(size_t)blockIdx.x * width + i] = from_f32<T>(((xr[i] * inv) * w[i]) / (1.0f + expf(-g)));
  }
}

template <typename T>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t s) {
  dim3 grid(n_seqs, a.heads, ceil_div(a.dv, 32));
  const int r = ceil_div(a.dk, kWarps);
  if (r <= 4) lightning_scan_kernel<T, 4><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 8) lightning_scan_kernel<T, 8><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 16) lightning_scan_kernel<T, 16><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 32) lightning_scan_kernel<T, 32><<<grid, kWarps * 32, 0, s>>>(a);
  else lightning_scan_kernel<T, 64><<<grid, kWarps * 32, 0, s>>>(a);
  return LMSF_LAUNCH_STATUS();
}

}  // namespace lmsf

// act: 0 none, 1 SiLU on q, k and v as they are read.  Strides in elements.
LMSF_API int lmsf_lightning_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                 long long v_stride, float* out, long long out_stride, float* state, const float* decay,
                                 const int* cu_q, const int* state_slot, int n_seqs, int heads, int dk, int dv, int act,
                                 int dtype, void* stream) {
  using namespace lmsf;
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dk > kMaxDk || dv <= 0)
    LMSF_REFUSE("lightning: heads=%d dk=%d dv=%d (dk up to %d)", heads, dk, dv, kMaxDk);
  if (ceil_div(dv, 32) > 65535) LMSF_REFUSE("lightning: dv=%d is too wide", dv);
  if (act != 0 && act != 1) LMSF_REFUSE("lightning: unknown activation code %d", act);
  ScanArgs a{q, k, v, q_stride, k_stride, v_stride, out, out_stride, state, decay, cu_q, state_slot, heads, dk, dv, act};
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) return launch_scan<float>(a, n_seqs, s);
  if (dtype == LMSF_BF16) return launch_scan<bf16>(a, n_seqs, s);
  LMSF_REFUSE("lightning: unknown dtype code %d", dtype);
}

LMSF_API int lmsf_gated_norm(void* out, const float* x, long long x_stride, const void* gate, long long gate_stride,
                             const float* w, int n, int width, float eps, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (width <= 0 || !(eps > 0.f)) LMSF_REFUSE("gated_norm: width=%d, eps must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) gated_norm_kernel<float><<<n, 256, 0, s>>>((float*)out, x, x_stride, (const float*)gate, gate_stride, w, width, eps);
  else if (dtype == LMSF_BF16) gated_norm_kernel<bf16><<<n, 256, 0, s>>>((bf16*)out, x, x_stride, (const bf16*)gate, gate_stride, w, width, eps);
  else LMSF_REFUSE("gated_norm: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}
