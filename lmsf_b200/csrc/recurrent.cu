// Recurrent mixers whose per-request state is one [dk, dv] matrix per head that every token decays, writes and reads
// (selective state-space layers with a scalar decay per head and token; the gated delta rule), and what stands around
// them: the short causal convolution over time with its carried inputs, and the norm over groups of columns with a gate.
//
//   causal_conv   y[t, c] = act(b[c] + sum_j w[c, j] * x[t - (taps - 1) + j, c]); inputs before a portion's first token
//                 come from the request's state slot ([taps - 1, channels] float32), which is rolled on afterwards
//   gated_scan    per request, head and token, in this order:
//                   dt = softplus(raw_dt + dt_bias[h]);  a = exp(-exp(a_log[h]) * dt)
//                   plain rule:  S <- a S + (dt k) v^T                      (k_times_dt; the write is k v^T without it)
//                   delta rule:  S <- a S;  u = sigmoid(raw_beta) (v - S^T k);  S <- S + k u^T
//                   o = S^T q (+ skip[h] v)
//                 q and k may be made unit vectors first (x / sqrt(sum x^2 + eps), q times a constant); several heads may
//                 share one q/k head.  The state, the decays and every sum are float32; the order of the sums does not
//                 depend on how a request's tokens are cut into steps.
//   grouped_gated_norm   out = norm_g(x) * w * act(gate)   or   out = norm_g(x * act(gate)) * w, the root mean square
//                 taken over each group of `gsize` columns, the weight indexed by column modulo its length
//
// The state of a head is stored transposed, [dv][dk]: the eight threads that share a column read consecutive rows.
// The scan is two launches: scan_prepare (per token: q and k scaled into the scan's layout, decay, write strength, step
// size) and the scan itself, whose blocks stage chunks of tokens by plain copies.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_recurrent)

namespace lmsf {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------- convolution

constexpr int kConvChannels = 64;    // channels per block (threadIdx.x)
constexpr int kConvChunk = 256;      // tokens per block along gridDim.z
constexpr int kMaxTaps = 8;

// grid (channel tiles, requests, token chunks); block (64, lanes): lanes of tokens side by side.
// Only the block of a request's first chunk reads its state, and only that block writes it (after its outputs):
// later chunks start at least kConvChunk >= taps - 1 tokens into the portion.
template <typename T>
__global__ void causal_conv_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                                   const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ state,
                                   long long slot_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                                   int C, int taps, int act) {
  const int c = blockIdx.x * kConvChannels + threadIdx.x;
  const int s = blockIdx.y;
  const int t0 = cu_q[s], n = cu_q[s + 1] - t0;
  const int lo = blockIdx.z * kConvChunk;
  if (lo >= n) return;
  const int hi = min(n, lo + kConvChunk);
  float* st = state + (size_t)state_slot[s] * slot_stride;      // [taps - 1][C]
  if (c < C) {
    float wr[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) wr[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    const float b = bias ? bias[c] : 0.f;
    for (int t = lo + threadIdx.y; t < hi; t += blockDim.y) {
      float acc = b;
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j) {
        if (j < taps) {
          const int u = t - (taps - 1) + j;                     // place in the portion; negative: before it
          const float v = u >= 0 ? to_f32(x[(size_t)(t0 + u) * x_stride + c]) : st[(size_t)(taps - 1 + u) * C + c];
          acc = fmaf(wr[j], v, acc);
        }
      }
      out[(size_t)(t0 + t) * out_stride + c] = from_f32<T>(act ? silu_f(acc) : acc);
    }
  }
  if (blockIdx.z != 0) return;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    // the last taps - 1 inputs, oldest first; row i reads row i + n of the old state (n >= 1: never a row already written)
    for (int i = 0; i < taps - 1; ++i) {
      const int u = n - (taps - 1) + i;
      const float v = u >= 0 ? to_f32(x[(size_t)(t0 + u) * x_stride + c]) : st[(size_t)(taps - 1 + u) * C + c];
      st[(size_t)i * C + c] = v;
    }
  }
}

// The same with VEC channels per thread (one 16-byte access of the activation type) and a window that slides in
// registers: a thread owns its channels for a chunk of kConvVecChunk tokens, reads every input once (and taps - 1 rows
// before the chunk), and, in a request's first chunk, is also the only reader and writer of its channels' state.
constexpr int kConvVecChunk = 32;
constexpr int kConvVecThreads = 128;

template <typename T, int VEC> __device__ __forceinline__ void conv_load(const T* p, float (&v)[VEC]);
template <> __device__ __forceinline__ void conv_load<float, 4>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void conv_load<bf16, 8>(const bf16* p, float (&v)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}
template <typename T, int VEC> __device__ __forceinline__ void conv_store(T* p, const float (&v)[VEC]);
template <> __device__ __forceinline__ void conv_store<float, 4>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void conv_store<bf16, 8>(bf16* p, const float (&v)[8]) {
  uint4 x;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = x;
}

template <typename T, int VEC, int TAPS>
__global__ void __launch_bounds__(kConvVecThreads) causal_conv_vec_kernel(
    T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
    const float* __restrict__ bias, float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_q,
    const int* __restrict__ state_slot, int C, int act) {
  const int c = (blockIdx.x * kConvVecThreads + threadIdx.x) * VEC;
  const int s = blockIdx.y;
  const int t0 = cu_q[s], n = cu_q[s + 1] - t0;
  const int lo = blockIdx.z * kConvVecChunk;
  if (lo >= n || c >= C) return;
  const int hi = min(n, lo + kConvVecChunk);
  float* st = state + (size_t)state_slot[s] * slot_stride;      // [TAPS - 1][C]
  float wr[TAPS][VEC], b[VEC], win[TAPS > 1 ? TAPS - 1 : 1][VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    b[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wr[j][e] = w[(size_t)(c + e) * TAPS + j];
  }
  // the TAPS - 1 inputs before the chunk, oldest first: from the portion, or (before its first token) from the state
#pragma unroll
  for (int j = 0; j < TAPS - 1; ++j) {
    const int u = lo - (TAPS - 1) + j;
    if (u >= 0) conv_load<T, VEC>(x + (size_t)(t0 + u) * x_stride + c, win[j]);
    else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) win[j][e] = st[(size_t)(TAPS - 1 + u) * C + c + e];
    }
  }
#pragma unroll 8
  for (int t = lo; t < hi; ++t) {
    float cur[VEC], acc[VEC];
    conv_load<T, VEC>(x + (size_t)(t0 + t) * x_stride + c, cur);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float a = b[e];
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) a = fmaf(wr[j][e], win[j][e], a);
      a = fmaf(wr[TAPS - 1][e], cur[e], a);
      acc[e] = act ? silu_f(a) : a;
    }
    conv_store<T, VEC>(out + (size_t)(t0 + t) * out_stride + c, acc);
#pragma unroll
    for (int j = 0; j + 1 < TAPS - 1; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) win[j][e] = win[j + 1][e];
    if (TAPS > 1) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) win[TAPS - 2][e] = cur[e];
    }
  }
  if (blockIdx.z != 0 || TAPS == 1) return;
  // the request's first chunk also rolls the state on (this thread alone reads and writes these channels of it)
  if (n <= kConvVecChunk) {                        // the window now holds the last TAPS - 1 inputs
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) st[(size_t)j * C + c + e] = win[j][e];
  } else {                                         // they lie at the end of the portion (n > TAPS - 1)
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {
      float v[VEC];
      conv_load<T, VEC>(x + (size_t)(t0 + n - (TAPS - 1) + j) * x_stride + c, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) st[(size_t)j * C + c + e] = v[e];
    }
  }
}

template <typename T, int VEC>
static int launch_conv_vec(void* out, long long out_stride, const void* x, long long x_stride, const float* w, const float* bias,
                           float* state, long long slot_stride, const int* cu_q, const int* state_slot, int n_seqs, int max_q, int C,
                           int taps, int act, cudaStream_t s) {
  dim3 grid(ceil_div(C, VEC * kConvVecThreads), n_seqs, ceil_div(max_q, kConvVecChunk));
#define LMSF_CASE(TP) case TP: causal_conv_vec_kernel<T, VEC, TP><<<grid, kConvVecThreads, 0, s>>>((T*)out, out_stride, (const T*)x, x_stride, w, bias, state, slot_stride, cu_q, state_slot, C, act); break;
  switch (taps) { LMSF_CASE(1) LMSF_CASE(2) LMSF_CASE(3) LMSF_CASE(4) LMSF_CASE(5) LMSF_CASE(6) LMSF_CASE(7) LMSF_CASE(8) default: return LMSF_EBADARG; }
#undef LMSF_CASE
  return LMSF_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------- scan

struct ScanArgs {
  float* out; long long out_stride;                            // [n, H * dv]
  const void* q; const void* k; const void* v;                 // q, k: [n, G * dk]; v: [n, H * dv]
  long long q_stride, k_stride, v_stride;
  const void* dt; long long dt_stride;                         // [n, H] raw step sizes
  const void* beta; long long beta_stride;                     // [n, H] raw write strengths (delta rule) or null
  const float* dt_bias; const float* a_log; const float* skip; // [H]; skip may be null
  float* state; long long slot_stride;                         // per slot [H][dv][dk] at the start
  const int* cu_q; const int* state_slot;
  int H, G, dk, dv;
  int k_times_dt, unit_qk;
  float unit_eps, q_scale;
  float* qf; float* kf; float4* gates;                         // what scan_prepare leaves for the scan (below)
  int n_tokens;
};

constexpr int kScanCols = 32;       // columns of the state per block
constexpr int kScanLanes = 8;       // threads that share a column: thread = (column c = tid / 8, row lane r = tid % 8)

// Row i = r + 8 m of a q or k vector lies at ((m / 4) * 8 + r) * 4 + m % 4 of its staged row of `rl` floats: the values
// m = 4 j .. 4 j + 3 of lane r are one 16-byte word, and the eight lanes of a column read consecutive words.
__device__ __forceinline__ int scan_place(int i) {
  const int r = i & 7, m = i >> 3;
  return ((m >> 2) * 8 + r) * 4 + (m & 3);
}

// Before the scan, once per token: q and k of every q/k head as float32 in the scan's own layout (made unit vectors and
// scaled, if asked; zero beyond dk), and per head the token's decay, write strength and step size.  A warp per (token,
// q/k head); the scan then stages its chunks by plain 16-byte copies that do not wait on each other.
template <typename T>
__global__ void __launch_bounds__(128) scan_prepare_kernel(ScanArgs a, int rl) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int g = warp; g < a.G; g += 4) {
    const T* qp = (const T*)a.q + (size_t)t * a.q_stride + (size_t)g * a.dk;
    const T* kp = (const T*)a.k + (size_t)t * a.k_stride + (size_t)g * a.dk;
    float fq = 1.f, fk = 1.f;
    if (a.unit_qk) {
      float ssq = 0.f, ssk = 0.f;
      for (int i = lane; i < a.dk; i += 32) {
        const float x = to_f32(qp[i]), y = to_f32(kp[i]);
        ssq = fmaf(x, x, ssq);
        ssk = fmaf(y, y, ssk);
      }
      ssq = warp_sum(ssq);
      ssk = warp_sum(ssk);
      fq = a.q_scale / sqrtf(ssq + a.unit_eps);
      fk = 1.0f / sqrtf(ssk + a.unit_eps);
    }
    float* qo = a.qf + ((size_t)t * a.G + g) * rl;
    float* ko = a.kf + ((size_t)t * a.G + g) * rl;
    for (int i = lane; i < rl; i += 32) {
      const int at = scan_place(i);
      qo[at] = i < a.dk ? to_f32(qp[i]) * fq : 0.f;
      ko[at] = i < a.dk ? to_f32(kp[i]) * fk : 0.f;
    }
  }
  for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
    const float dt = softplus_f(to_f32(((const T*)a.dt)[(size_t)t * a.dt_stride + h]) + a.dt_bias[h]);
    const float dec = expf(-expf(a.a_log[h]) * dt);
    const float beta = a.beta ? sigmoid_f(to_f32(((const T*)a.beta)[(size_t)t * a.beta_stride + h])) : 1.f;
    a.gates[(size_t)t * a.H + h] = make_float4(dec, beta, a.k_times_dt ? dt : 1.f, 0.f);
  }
}

// grid (column tiles, heads, requests); 256 threads; rows r + 8 m of a column in registers.  A chunk of tokens is staged
// in shared memory; sums over the rows run in four chains that are added at the end, then over the eight lanes by a
// butterfly (a fixed order).
template <typename T, int ROWS, bool DELTA>
__global__ void __launch_bounds__(256) gated_scan_kernel(ScanArgs a) {
  constexpr int R = kScanLanes, COLS = kScanCols;
  constexpr int RV = (ROWS + 3) / 4;              // 16-byte words per lane and row
  constexpr int RL = RV * 4 * R;                  // floats of a staged row
  constexpr int CH = RL <= 128 ? 32 : 16;         // tokens staged at a time
  __shared__ __align__(16) float sq[CH][RL];
  __shared__ __align__(16) float sk[CH][RL];
  __shared__ float sv[CH][COLS];
  __shared__ float4 sg[CH];
  const int tid = threadIdx.x, c = tid / R, r = tid % R;
  const int head = blockIdx.y, seq = blockIdx.z, col = blockIdx.x * COLS + c;
  const int g = head / (a.H / a.G);
  const int t0 = a.cu_q[seq], n = a.cu_q[seq + 1] - t0;
  if (n <= 0) return;
  float* st = a.state + (size_t)a.state_slot[seq] * a.slot_stride + (size_t)head * a.dv * a.dk;
  const bool live = col < a.dv;
  float S[ROWS];
#pragma unroll
  for (int m = 0; m < ROWS; ++m) {
    const int i = r + R * m;
    S[m] = (live && i < a.dk) ? st[(size_t)col * a.dk + i] : 0.f;
  }
  const float skip = a.skip ? a.skip[head] : 0.f;
  for (int base = 0; base < n; base += CH) {
    const int cnt = min(CH, n - base);
    __syncthreads();
    for (int idx = tid; idx < cnt * (RL / 4); idx += 256) {
      const int tt = idx / (RL / 4), w4 = idx % (RL / 4);
      const size_t row = ((size_t)(t0 + base + tt) * a.G + g) * RL;
      *reinterpret_cast<float4*>(&sq[tt][4 * w4]) = *reinterpret_cast<const float4*>(a.qf + row + 4 * w4);
      *reinterpret_cast<float4*>(&sk[tt][4 * w4]) = *reinterpret_cast<const float4*>(a.kf + row + 4 * w4);
    }
    for (int idx = tid; idx < cnt * COLS; idx += 256) {
      const int tt = idx / COLS, cc = blockIdx.x * COLS + idx % COLS;
      sv[tt][idx % COLS] = cc < a.dv ? to_f32(((const T*)a.v)[(size_t)(t0 + base + tt) * a.v_stride + (size_t)head * a.dv + cc]) : 0.f;
    }
    if (tid < cnt) sg[tid] = a.gates[(size_t)(t0 + base + tid) * a.H + head];
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float4 gt = sg[tt];                   // decay, write strength, step size
      const float dec = gt.x, vv = sv[tt][c];
      float kk[RV * 4], qq[RV * 4];
#pragma unroll
      for (int j = 0; j < RV; ++j) {
        const float4 x = *reinterpret_cast<const float4*>(&sk[tt][(j * R + r) * 4]);
        const float4 y = *reinterpret_cast<const float4*>(&sq[tt][(j * R + r) * 4]);
        kk[4 * j] = x.x; kk[4 * j + 1] = x.y; kk[4 * j + 2] = x.z; kk[4 * j + 3] = x.w;
        qq[4 * j] = y.x; qq[4 * j + 1] = y.y; qq[4 * j + 2] = y.z; qq[4 * j + 3] = y.w;
      }
      float u = gt.z * vv;                        // the plain rule writes (dt k) v^T = k (dt v)^T
      if (DELTA) {
        float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
          S[m] *= dec;
          p[m & 3] = fmaf(S[m], kk[m], p[m & 3]);
        }
        float ps = (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
        for (int off = R / 2; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        u = gt.y * (vv - ps);
      }
      float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        S[m] = DELTA ? fmaf(kk[m], u, S[m]) : fmaf(kk[m], u, dec * S[m]);
        o[m & 3] = fmaf(S[m], qq[m], o[m & 3]);
      }
      float os = (o[0] + o[1]) + (o[2] + o[3]);
#pragma unroll
      for (int off = R / 2; off > 0; off >>= 1) os += __shfl_xor_sync(0xffffffffu, os, off);
      if (r == 0 && live) a.out[(size_t)(t0 + base + tt) * a.out_stride + (size_t)head * a.dv + col] = fmaf(skip, vv, os);
    }
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      const int i = r + R * m;
      if (i < a.dk) st[(size_t)col * a.dk + i] = S[m];
    }
  }
}

static int scan_rows(int dk) {                     // rows per lane, as the kernel is built: 2, 4, 8, 16 or 32
  const int rows = ceil_div(dk, kScanLanes);
  return rows <= 2 ? 2 : rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
}
static int scan_row_floats(int dk) { return (scan_rows(dk) + 3) / 4 * 4 * kScanLanes; }

template <typename T, bool DELTA>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t s) {
  scan_prepare_kernel<T><<<a.n_tokens, 128, 0, s>>>(a, scan_row_floats(a.dk));
  dim3 grid(ceil_div(a.dv, kScanCols), a.H, n_seqs);
  switch (scan_rows(a.dk)) {
    case 2: gated_scan_kernel<T, 2, DELTA><<<grid, 256, 0, s>>>(a); break;
    case 4: gated_scan_kernel<T, 4, DELTA><<<grid, 256, 0, s>>>(a); break;
    case 8: gated_scan_kernel<T, 8, DELTA><<<grid, 256, 0, s>>>(a); break;
    case 16: gated_scan_kernel<T, 16, DELTA><<<grid, 256, 0, s>>>(a); break;
    default: gated_scan_kernel<T, 32, DELTA><<<grid, 256, 0, s>>>(a); break;
  }
  return LMSF_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------------------------- norm over groups

// A team (a warp, or the whole block) serves one (token, group).
template <typename T, bool BLOCK>
__global__ void grouped_gated_norm_kernel(T* __restrict__ out, long long out_stride, const float* __restrict__ x,
                                          long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                          const float* __restrict__ w, int wlen, int n, int n_groups, int gsize, float eps,
                                          int gate_silu, int gate_first) {
  __shared__ float scratch[33];
  const int team = BLOCK ? blockIdx.x : blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int me = BLOCK ? threadIdx.x : (threadIdx.x & 31), step = BLOCK ? blockDim.x : 32;
  if (team >= n * n_groups) return;
  const int t = team / n_groups, grp = team % n_groups;
  const float* xr = x + (size_t)t * x_stride + (size_t)grp * gsize;
  const T* gr = gate ? gate + (size_t)t * gate_stride + (size_t)grp * gsize : nullptr;
  float ss = 0.f;
  for (int i = me; i < gsize; i += step) {
    float v = xr[i];
    if (gate_first && gr) { const float z = to_f32(gr[i]); v *= gate_silu ? silu_f(z) : sigmoid_f(z); }
    ss = fmaf(v, v, ss);
  }
  ss = BLOCK ? block_sum(ss, scratch) : warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)gsize + eps);
  T* o = out + (size_t)t * out_stride + (size_t)grp * gsize;
  for (int i = me; i < gsize; i += step) {
    float v = xr[i];
    const float z = gr ? to_f32(gr[i]) : 0.f;
    const float gv = gr ? (gate_silu ? silu_f(z) : sigmoid_f(z)) : 1.f;
    if (gate_first) v *= gv;
    v = (v * inv) * w[(grp * gsize + i) % wlen];
    if (!gate_first) v *= gv;
    o[i] = from_f32<T>(v);
  }
}

// The same with a group's values held in registers between the sum of squares and the scaling (PER accesses of V values
// per member of the team): x and the gate are read once.  V = 4: 16-byte reads of x, 8- or 16-byte accesses of the gate
// and the output (the group's size, the weight's length and the row strides are multiples of 4, the pointers aligned).
template <typename T, int V> struct alignas(sizeof(T) * V) NormVec { T v[V]; };

template <typename T, bool BLOCK, int PER, int V>
__global__ void __launch_bounds__(BLOCK ? 256 : 128) grouped_gated_norm_reg_kernel(
    T* __restrict__ out, long long out_stride, const float* __restrict__ x, long long x_stride, const T* __restrict__ gate,
    long long gate_stride, const float* __restrict__ w, int wlen, int n, int n_groups, int gsize, float eps, int gate_silu,
    int gate_first) {
  __shared__ float scratch[33];
  const int team = BLOCK ? blockIdx.x : blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int me = BLOCK ? threadIdx.x : (threadIdx.x & 31), step = BLOCK ? 256 : 32;
  if (team >= n * n_groups) return;
  const int t = team / n_groups, grp = team % n_groups;
  const float* xr = x + (size_t)t * x_stride + (size_t)grp * gsize;
  const T* gr = gate ? gate + (size_t)t * gate_stride + (size_t)grp * gsize : nullptr;
  float v[PER][V], gv[PER][V];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = (me + step * j) * V;
    NormVec<float, V> xv;
    NormVec<T, V> zv;
    if (i < gsize) {
      xv = *reinterpret_cast<const NormVec<float, V>*>(xr + i);
      if (gr) zv = *reinterpret_cast<const NormVec<T, V>*>(gr + i);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      v[j][e] = i < gsize ? xv.v[e] : 0.f;
      gv[j][e] = 1.f;
      if (gr && i < gsize) { const float z = to_f32(zv.v[e]); gv[j][e] = gate_silu ? silu_f(z) : sigmoid_f(z); }
      if (gate_first) v[j][e] *= gv[j][e];
      ss = fmaf(v[j][e], v[j][e], ss);
    }
  }
  ss = BLOCK ? block_sum(ss, scratch) : warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)gsize + eps);
  T* o = out + (size_t)t * out_stride + (size_t)grp * gsize;
  const int w0 = (int)(((long long)grp * gsize) % wlen);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = (me + step * j) * V;
    if (i < gsize) {
      int wi = w0 + i;                              // the weight repeats after wlen columns
      if (wi >= wlen) wi %= wlen;
      NormVec<T, V> ov;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float r = (v[j][e] * inv) * w[wi + e];
        if (!gate_first) r *= gv[j][e];
        ov.v[e] = from_f32<T>(r);
      }
      *reinterpret_cast<NormVec<T, V>*>(o + i) = ov;
    }
  }
}

}  // namespace lmsf

// x: [n, C] rows of `dtype` with x_stride elements between tokens; out likewise; w: float32 [C, taps]; bias: float32 [C] or
// null; state: float32, the [taps - 1, C] block of slot s starts at state + s * slot_stride.  act: 0 none, 1 silu.
// max_q: the longest portion of the launch (the host's copy; sizes the grid only).
LMSF_API int lmsf_causal_conv(void* out, long long out_stride, const void* x, long long x_stride, const float* w,
                              const float* bias, float* state, long long slot_stride, const int* cu_q, const int* state_slot,
                              int n_seqs, int max_q, int C, int taps, int act, int dtype, void* stream) {
  using namespace lmsf;
  if (n_seqs <= 0 || max_q <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > kMaxTaps) LMSF_REFUSE("causal_conv: %d channels, %d taps (1 to %d taps)", C, taps, kMaxTaps);
  if (n_seqs > 65535) LMSF_REFUSE("causal_conv: more than 65535 requests in one launch");
  cudaStream_t s = (cudaStream_t)stream;
  if (ceil_div(max_q, kConvVecChunk) > 65535) LMSF_REFUSE("causal_conv: a portion of %d tokens is too long for one launch", max_q);
  // 16-byte accesses where the rows allow them (the state's rows are then 16-byte aligned too)
  const int vec = dtype == LMSF_F32 ? 4 : 8;
  if ((dtype == LMSF_F32 || dtype == LMSF_BF16) && C % vec == 0 && out_stride % vec == 0 && x_stride % vec == 0 &&
      ((uintptr_t)out | (uintptr_t)x) % 16 == 0) {
    if (dtype == LMSF_F32) return launch_conv_vec<float, 4>(out, out_stride, x, x_stride, w, bias, state, slot_stride, cu_q, state_slot, n_seqs, max_q, C, taps, act, s);
    return launch_conv_vec<bf16, 8>(out, out_stride, x, x_stride, w, bias, state, slot_stride, cu_q, state_slot, n_seqs, max_q, C, taps, act, s);
  }
  dim3 grid(ceil_div(C, kConvChannels), n_seqs, ceil_div(max_q, kConvChunk));
  dim3 block(kConvChannels, max_q >= 4 ? 4 : (max_q >= 2 ? 2 : 1));
  if (dtype == LMSF_F32)
    causal_conv_kernel<float><<<grid, block, 0, s>>>((float*)out, out_stride, (const float*)x, x_stride, w, bias, state, slot_stride, cu_q, state_slot, C, taps, act);
  else if (dtype == LMSF_BF16)
    causal_conv_kernel<bf16><<<grid, block, 0, s>>>((bf16*)out, out_stride, (const bf16*)x, x_stride, w, bias, state, slot_stride, cu_q, state_slot, C, taps, act);
  else LMSF_REFUSE("causal_conv: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// Floats of the scratch that lmsf_gated_scan needs for n_tokens tokens (q and k in the scan's layout, and four floats per
// token and head).
LMSF_API long long lmsf_gated_scan_scratch_floats(int n_tokens, int H, int G, int dk) {
  return (long long)n_tokens * (2LL * G * lmsf::scan_row_floats(dk) + 4LL * H);
}

LMSF_API int lmsf_gated_scan(float* out, long long out_stride, const void* q, const void* k, const void* v, long long q_stride,
                             long long k_stride, long long v_stride, const void* dt, long long dt_stride, const void* beta,
                             long long beta_stride, const float* dt_bias, const float* a_log, const float* skip, float* state,
                             long long slot_stride, const int* cu_q, const int* state_slot, int n_seqs, int n_tokens, int H,
                             int G, int dk, int dv, int delta, int k_times_dt, int unit_qk, float unit_eps, float q_scale,
                             float* scratch, int dtype, void* stream) {
  using namespace lmsf;
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dk <= 0 || dk > 256 || dv <= 0 || H > 65535 || n_seqs > 65535)
    LMSF_REFUSE("gated_scan: %d heads over %d q/k heads, dk=%d (up to 256), dv=%d", H, G, dk, dv);
  if (delta && !beta) LMSF_REFUSE("gated_scan: the delta rule needs a write strength per head and token");
  if (!scratch || (uintptr_t)scratch % 16) LMSF_REFUSE("gated_scan: a 16-byte aligned scratch is needed");
  const long long rowf = (long long)n_tokens * G * scan_row_floats(dk);
  ScanArgs a{out, out_stride, q, k, v, q_stride, k_stride, v_stride, dt, dt_stride, beta, beta_stride, dt_bias, a_log, skip,
             state, slot_stride, cu_q, state_slot, H, G, dk, dv, k_times_dt, unit_qk, unit_eps, q_scale,
             scratch, scratch + rowf, reinterpret_cast<float4*>(scratch + 2 * rowf), n_tokens};
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (dtype == LMSF_F32) rc = delta ? launch_scan<float, true>(a, n_seqs, s) : launch_scan<float, false>(a, n_seqs, s);
  else if (dtype == LMSF_BF16) rc = delta ? launch_scan<bf16, true>(a, n_seqs, s) : launch_scan<bf16, false>(a, n_seqs, s);
  else LMSF_REFUSE("gated_scan: unknown dtype code %d", dtype);
  return rc;
}

// x: float32 [n, n_groups * gsize]; gate (may be null) and out: rows of `dtype`; w: float32 [wlen], wlen divides into the row.
LMSF_API int lmsf_grouped_gated_norm(void* out, long long out_stride, const float* x, long long x_stride, const void* gate,
                                     long long gate_stride, const float* w, int wlen, int n, int n_groups, int gsize, float eps,
                                     int gate_silu, int gate_first, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (n_groups <= 0 || gsize <= 0 || wlen <= 0 || !(eps > 0.f)) LMSF_REFUSE("grouped_gated_norm: %d groups of %d, eps %g", n_groups, gsize, eps);
  cudaStream_t s = (cudaStream_t)stream;
  const long long teams = (long long)n * n_groups;
  const bool block = gsize > 1024;
  const unsigned blocks = (unsigned)(block ? teams : (teams + 3) / 4);
  const size_t esz = dtype == LMSF_F32 ? 4 : 2;
  const bool wide = gsize % 4 == 0 && wlen % 4 == 0 && x_stride % 4 == 0 && out_stride % 4 == 0 && (!gate || gate_stride % 4 == 0) &&
                    ((uintptr_t)x | (uintptr_t)w) % 16 == 0 && ((uintptr_t)out | (uintptr_t)gate) % (4 * esz) == 0;
  const int per = ceil_div(gsize, (block ? 256 : 32) * (wide ? 4 : 1));
#define LMSF_REG(T, B, P, V) grouped_gated_norm_reg_kernel<T, B, P, V><<<blocks, B ? 256 : 128, 0, s>>>((T*)out, out_stride, x, x_stride, (const T*)gate, gate_stride, w, wlen, n, n_groups, gsize, eps, gate_silu, gate_first)
#define LMSF_CASE(T, B, P) if (per <= P) { if (wide) LMSF_REG(T, B, P, 4); else LMSF_REG(T, B, P, 1); return LMSF_LAUNCH_STATUS(); }
#define LMSF_NARROW(T, B, P) if (!wide && per <= P) { LMSF_REG(T, B, P, 1); return LMSF_LAUNCH_STATUS(); }
#define LMSF_PICK(T)                                                                          \
  if (!block) { LMSF_CASE(T, false, 1) LMSF_CASE(T, false, 2) LMSF_CASE(T, false, 4) LMSF_CASE(T, false, 8)  \
                LMSF_NARROW(T, false, 16) LMSF_NARROW(T, false, 32) }                          \
  else { LMSF_CASE(T, true, 2) LMSF_CASE(T, true, 4) LMSF_NARROW(T, true, 8) LMSF_NARROW(T, true, 16) LMSF_NARROW(T, true, 32) }
  if (dtype == LMSF_F32) { LMSF_PICK(float) }
  else if (dtype == LMSF_BF16) { LMSF_PICK(bf16) }
#undef LMSF_PICK
#undef LMSF_NARROW
#undef LMSF_CASE
#undef LMSF_REG
#define LMSF_GO(T, B) grouped_gated_norm_kernel<T, B><<<blocks, B ? 256 : 128, 0, s>>>((T*)out, out_stride, x, x_stride, (const T*)gate, gate_stride, w, wlen, n, n_groups, gsize, eps, gate_silu, gate_first)
  if (dtype == LMSF_F32) { if (block) LMSF_GO(float, true); else LMSF_GO(float, false); }
  else if (dtype == LMSF_BF16) { if (block) LMSF_GO(bf16, true); else LMSF_GO(bf16, false); }
  else LMSF_REFUSE("grouped_gated_norm: unknown dtype code %d", dtype);
#undef LMSF_GO
  return LMSF_LAUNCH_STATUS();
}
