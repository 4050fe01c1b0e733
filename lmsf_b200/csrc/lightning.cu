// Linear attention with a decay per head ("lightning attention") and the gated norm that follows it.
//
//   S_t = a_h S_(t-1) + k_t v_t^T      (S: [dk, dv] per request and head, float32, kept across steps in a state slot)
//   o_t = S_t^T q_t
//
// q, k, v arrive as the rows of a projection's output and pass through an activation on the way in (SiLU or none),
// computed in float32 from the stored value; the state, the decay and the output are float32 throughout.
//
// lightning_scan_kernel: one block per (request, head, 64 value columns).  Warp w holds rows [w R, (w + 1) R) of the
// state's 64 columns in registers (two columns per lane); the request's tokens are taken in chunks of kChunk whose
// q, k and v rows are staged in shared memory (activation applied, four values per read where the rows allow it; a
// 16-byte shared-memory read of q or k then serves four rows of both columns of every lane);
// every warp walks the chunk token by token and leaves its partial
// outputs in shared memory, which are added up in a fixed order after the chunk.  A request that brings one token
// (a decode step) runs the same code with one chunk of one token: the state is read and written once.
// Portions of up to a few hundred tokens perform the same operations on the state in the same order however the
// sequence is cut, so their results do not depend on the cut by a bit.
//
// Long portions (a prompt) would leave most of the device idle behind one request's chain of tokens.  They are cut into
// chunks that run in parallel, in two passes of the same kernel: pass 1 runs every chunk from a ZERO state and keeps the
// state it ends with; a small kernel then walks each request's chunks in order, S_before(c + 1) = decay^n S_before(c) +
// added(c), which is exact because the recurrence is linear in the state; pass 2 runs every chunk again from its true
// state and writes the outputs.  Twice the arithmetic, all of it float32 FMA as before, on all SMs.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_lightning)

namespace lmsf {

constexpr int kWarps = 4;
constexpr int kMaxDk = 256;
constexpr int kCols = 64;    // value columns of the state per block: two per lane

__device__ __forceinline__ float act_in(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }

struct ScanArgs {
  const void* q; const void* k; const void* v;     // rows of [n_tokens, *]; head h starts at h * dk (q, k) or h * dv (v)
  long long q_stride, k_stride, v_stride;
  float* out; long long out_stride;                // [n_tokens, heads * dv] float32
  float* state;                                    // [slots, heads, dk, dv] float32
  const float* decay;                              // [heads]
  const int* cu_q; const int* state_slot;          // [n_seqs + 1], [n_seqs]
  int heads, dk, dv, act;
  const int4* items;                               // work items (request, first token, end token, index in scratch); null: item i is request i, whole
  float* scratch;                                  // [items of modes 1 and 2][heads][dk][dv] float32
};

// MODE 0: a request's tokens of this step in order, state read from and written to its slot.
// MODE 1: one chunk of a long portion from a ZERO state; the state it ends with goes to scratch[item] (no outputs).
// MODE 2: one chunk from the state that scratch[item] holds (what the request's state was before the chunk); outputs only.
// four consecutive activations of a row as floats (one 8- or 16-byte read)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int R, int MODE>
__global__ void __launch_bounds__(kWarps * 32) lightning_scan_kernel(ScanArgs a) {
  constexpr int kRows = kWarps * R;                  // rows of the state that the block walks (>= dk; the rest are zeros)
  constexpr int kChunk = R > 32 ? 8 : 16;            // tokens staged at a time (shared memory stays under 48 KB)
  __shared__ __align__(16) float qs[MODE == 1 ? 1 : kChunk][kRows];
  __shared__ __align__(16) float ks[kChunk][kRows];
  __shared__ __align__(16) float vs[kChunk][kCols];
  __shared__ float part[MODE == 1 ? 1 : kWarps][kChunk][kCols];
  const int head = blockIdx.y, col0 = blockIdx.z * kCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int seq = blockIdx.x, t0, t1, slot_item = 0;
  if (a.items != nullptr) {
    const int4 it = a.items[blockIdx.x];
    seq = it.x; t0 = it.y; t1 = it.z; slot_item = it.w;
  } else {
    t0 = a.cu_q[seq]; t1 = a.cu_q[seq + 1];
  }
  if (t1 <= t0) return;
  const int dk = a.dk, dv = a.dv;
  const int cA = col0 + lane, cB = col0 + 32 + lane;   // a lane's two columns of the state
  const bool liveA = cA < dv, liveB = cB < dv;
  const float decay = a.decay[head];
  float* st = MODE == 0 ? a.state + (((size_t)a.state_slot[seq] * a.heads + head) * dk) * dv
                        : a.scratch + (((size_t)slot_item * a.heads + head) * dk) * dv;
  const int r0 = warp * R;
  float SA[R], SB[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    SA[i] = (MODE != 1 && liveA && r0 + i < dk) ? st[(size_t)(r0 + i) * dv + cA] : 0.f;
    SB[i] = (MODE != 1 && liveB && r0 + i < dk) ? st[(size_t)(r0 + i) * dv + cB] : 0.f;
  }
  const T* qg = (const T*)a.q + (size_t)head * dk;
  const T* kg = (const T*)a.k + (size_t)head * dk;
  const T* vg = (const T*)a.v + (size_t)head * dv + col0;
  // rows may be read four values at a time when every row and head starts on such a boundary
  const bool wide_qk = dk % 4 == 0 && a.q_stride % 4 == 0 && a.k_stride % 4 == 0 && ((uintptr_t)a.q | (uintptr_t)a.k) % (4 * sizeof(T)) == 0;
  const bool wide_v = dv % 4 == 0 && a.v_stride % 4 == 0 && (uintptr_t)a.v % (4 * sizeof(T)) == 0;

  for (int c0 = t0; c0 < t1; c0 += kChunk) {
    const int n = min(kChunk, t1 - c0);
    __syncthreads();   // the chunk before has been read
    if (wide_qk) {
      for (int e = threadIdx.x; e < n * (kRows / 4); e += kWarps * 32) {
        const int t = e / (kRows / 4), d = (e - t * (kRows / 4)) * 4;
        float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), qq = kk;
        if (d < dk) {
          kk = ld4(kg + (size_t)(c0 + t) * a.k_stride + d);
          kk = make_float4(act_in(kk.x, a.act), act_in(kk.y, a.act), act_in(kk.z, a.act), act_in(kk.w, a.act));
          if (MODE != 1) {
            qq = ld4(qg + (size_t)(c0 + t) * a.q_stride + d);
            qq = make_float4(act_in(qq.x, a.act), act_in(qq.y, a.act), act_in(qq.z, a.act), act_in(qq.w, a.act));
          }
        }
        *reinterpret_cast<float4*>(&ks[t][d]) = kk;
        if (MODE != 1) *reinterpret_cast<float4*>(&qs[t][d]) = qq;
      }
    } else {
      for (int e = threadIdx.x; e < n * kRows; e += kWarps * 32) {
        const int t = e / kRows, d = e - t * kRows;
        if (MODE != 1) qs[t][d] = d < dk ? act_in(to_f32(qg[(size_t)(c0 + t) * a.q_stride + d]), a.act) : 0.f;
        ks[t][d] = d < dk ? act_in(to_f32(kg[(size_t)(c0 + t) * a.k_stride + d]), a.act) : 0.f;
      }
    }
    if (wide_v) {
      for (int e = threadIdx.x; e < n * (kCols / 4); e += kWarps * 32) {
        const int t = e / (kCols / 4), c = (e - t * (kCols / 4)) * 4;
        float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col0 + c < dv) {
          vv = ld4(vg + (size_t)(c0 + t) * a.v_stride + c);
          vv = make_float4(act_in(vv.x, a.act), act_in(vv.y, a.act), act_in(vv.z, a.act), act_in(vv.w, a.act));
        }
        *reinterpret_cast<float4*>(&vs[t][c]) = vv;
      }
    } else {
      for (int e = threadIdx.x; e < n * kCols; e += kWarps * 32) {
        const int t = e / kCols, c = e - t * kCols;
        vs[t][c] = col0 + c < dv ? act_in(to_f32(vg[(size_t)(c0 + t) * a.v_stride + c]), a.act) : 0.f;
      }
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float vA = vs[t][lane], vB = vs[t][32 + lane];
      float oA = 0.f, oB = 0.f;
      const float4* k4 = reinterpret_cast<const float4*>(&ks[t][r0]);     // one 16-byte read serves four rows of every lane
      const float4* q4 = reinterpret_cast<const float4*>(&qs[MODE == 1 ? 0 : t][r0]);
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 kk = k4[i];
        SA[4 * i + 0] = fmaf(decay, SA[4 * i + 0], kk.x * vA);  SB[4 * i + 0] = fmaf(decay, SB[4 * i + 0], kk.x * vB);
        SA[4 * i + 1] = fmaf(decay, SA[4 * i + 1], kk.y * vA);  SB[4 * i + 1] = fmaf(decay, SB[4 * i + 1], kk.y * vB);
        SA[4 * i + 2] = fmaf(decay, SA[4 * i + 2], kk.z * vA);  SB[4 * i + 2] = fmaf(decay, SB[4 * i + 2], kk.z * vB);
        SA[4 * i + 3] = fmaf(decay, SA[4 * i + 3], kk.w * vA);  SB[4 * i + 3] = fmaf(decay, SB[4 * i + 3], kk.w * vB);
        if (MODE != 1) {
          const float4 qq = q4[i];
          oA = fmaf(qq.x, SA[4 * i + 0], oA);  oB = fmaf(qq.x, SB[4 * i + 0], oB);
          oA = fmaf(qq.y, SA[4 * i + 1], oA);  oB = fmaf(qq.y, SB[4 * i + 1], oB);
          oA = fmaf(qq.z, SA[4 * i + 2], oA);  oB = fmaf(qq.z, SB[4 * i + 2], oB);
          oA = fmaf(qq.w, SA[4 * i + 3], oA);  oB = fmaf(qq.w, SB[4 * i + 3], oB);
        }
      }
      if (MODE != 1) { part[warp][t][lane] = oA; part[warp][t][32 + lane] = oB; }
    }
    if (MODE == 1) continue;
    __syncthreads();
    for (int e = threadIdx.x; e < n * kCols; e += kWarps * 32) {
      const int t = e / kCols, l = e - t * kCols;
      if (col0 + l < dv) {
        float o = part[0][t][l];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) o += part[MODE == 1 ? 0 : w][t][l];
        a.out[(size_t)(c0 + t) * a.out_stride + (size_t)head * dv + col0 + l] = o;
      }
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (liveA && r0 + i < dk) st[(size_t)(r0 + i) * dv + cA] = SA[i];
      if (liveB && r0 + i < dk) st[(size_t)(r0 + i) * dv + cB] = SB[i];
    }
  }
}

// Between the two passes over the chunks of long portions: for every long portion (request, its chunks first..end in
// the item list) walk the chunks in order; scratch[c] holds what chunk c adds from a zero state and receives the state
// BEFORE chunk c; the state after the last chunk goes to the request's slot.  S_after = decay^tokens * S_before + added.
__global__ void lightning_prefix_kernel(float* __restrict__ scratch, float* __restrict__ state, const float* __restrict__ decay,
                                        const int* __restrict__ state_slot, const int4* __restrict__ items,
                                        const int4* __restrict__ spans, int heads, int per_head) {
  const int4 sp = spans[blockIdx.x];                 // (request, first chunk item, end chunk item, -)
  const int head = blockIdx.y;
  const float a = decay[head];
  const size_t per_item = (size_t)heads * per_head;
  float* slot = state + ((size_t)state_slot[sp.x] * heads + head) * per_head;
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < per_head; e += gridDim.z * blockDim.x) {
    float S = slot[e];
    for (int c = sp.y; c < sp.z; ++c) {
      const int4 it = items[c];
      float* cell = scratch + (size_t)it.w * per_item + (size_t)head * per_head + e;
      const float added = *cell;
      *cell = S;
      float p = 1.f;
      for (int t = it.y; t < it.z; ++t) p *= a;      // the same product of decays that the tokens would apply one by one
      S = fmaf(p, S, added);
    }
    slot[e] = S;
  }
}

// out[t] = norm(x[t]) * w * sigmoid(gate[t]) : the norm over all heads of a token together, float32 inside.
// x: float32 [n, width]; gate: rows of the activation type; out: activation type [n, width].  One block per token.
template <typename T, int V>
__global__ void __launch_bounds__(256) gated_norm_kernel(T* __restrict__ out, const float* __restrict__ x, long long x_stride,
                                                         const T* __restrict__ gate, long long gate_stride,
                                                         const float* __restrict__ w, int width, float eps) {
  __shared__ float scratch[33];
  const float* xr = x + (size_t)blockIdx.x * x_stride;
  const T* gr = gate + (size_t)blockIdx.x * gate_stride;
  T* orow = out + (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
    if (V == 4) { const float4 a = *reinterpret_cast<const float4*>(xr + i); ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss)))); }
    else ss = fmaf(xr[i], xr[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x * V; i < width; i += blockDim.x * V) {
    if (V == 4) {       // (second read of the row: it comes from cache)
      const float4 a = *reinterpret_cast<const float4*>(xr + i), ww = *reinterpret_cast<const float4*>(w + i);
      float g[4], o[4];
      if (sizeof(T) == 2) {
        const uint2 u = *reinterpret_cast<const uint2*>(gr + i);
        const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        g[0] = g0.x; g[1] = g0.y; g[2] = g1.x; g[3] = g1.y;
      } else {
        const float4 u = *reinterpret_cast<const float4*>(gr + i);
        g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
      }
      o[0] = ((a.x * inv) * ww.x) / (1.0f + expf(-g[0]));
      o[1] = ((a.y * inv) * ww.y) / (1.0f + expf(-g[1]));
      o[2] = ((a.z * inv) * ww.z) / (1.0f + expf(-g[2]));
      o[3] = ((a.w * inv) * ww.w) / (1.0f + expf(-g[3]));
      if (sizeof(T) == 2) {
        uint2 u;
        *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(o[0], o[1]);
        *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(o[2], o[3]);
        *reinterpret_cast<uint2*>(orow + i) = u;
      } else {
        *reinterpret_cast<float4*>(orow + i) = make_float4(o[0], o[1], o[2], o[3]);
      }
    } else {
      const float g = to_f32(gr[i]);
      orow[i] = from_f32<T>(((xr[i] * inv) * w[i]) / (1.0f + expf(-g)));
    }
  }
}

template <typename T, int MODE>
static int launch_scan(const ScanArgs& a, int n_items, cudaStream_t s) {
  dim3 grid(n_items, a.heads, ceil_div(a.dv, kCols));
  const int r = ceil_div(a.dk, kWarps);
  if (r <= 4) lightning_scan_kernel<T, 4, MODE><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 8) lightning_scan_kernel<T, 8, MODE><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 16) lightning_scan_kernel<T, 16, MODE><<<grid, kWarps * 32, 0, s>>>(a);
  else if (r <= 32) lightning_scan_kernel<T, 32, MODE><<<grid, kWarps * 32, 0, s>>>(a);
  else lightning_scan_kernel<T, 64, MODE><<<grid, kWarps * 32, 0, s>>>(a);
  return LMSF_LAUNCH_STATUS();
}

template <typename T>
static int launch_mode(const ScanArgs& a, int n_items, int mode, cudaStream_t s) {
  if (mode == 0) return launch_scan<T, 0>(a, n_items, s);
  if (mode == 1) return launch_scan<T, 1>(a, n_items, s);
  return launch_scan<T, 2>(a, n_items, s);
}

}  // namespace lmsf

// act: 0 none, 1 SiLU on q, k and v as they are read.  Strides in elements.
// items (int32 [n_items][4], may be null): (request, first token, end token, index in scratch) per block row; null: one item
// per request, its whole portion (what a decode step uses: nothing comes from the host).  mode 0: state in the slots;
// modes 1 and 2: the two passes over the chunks of long portions, with lmsf_lightning_prefix between them.
LMSF_API int lmsf_lightning_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                 long long v_stride, float* out, long long out_stride, float* state, const float* decay,
                                 const int* cu_q, const int* state_slot, int n_items, int heads, int dk, int dv, int act,
                                 int dtype, const int* items, float* scratch, int mode, void* stream) {
  using namespace lmsf;
  if (n_items <= 0) return 0;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dk > kMaxDk || dv <= 0)
    LMSF_REFUSE("lightning: heads=%d dk=%d dv=%d (dk up to %d)", heads, dk, dv, kMaxDk);
  if (ceil_div(dv, kCols) > 65535) LMSF_REFUSE("lightning: dv=%d is too wide", dv);
  if (act != 0 && act != 1) LMSF_REFUSE("lightning: unknown activation code %d", act);
  if (mode < 0 || mode > 2 || (mode != 0 && (items == nullptr || scratch == nullptr)))
    LMSF_REFUSE("lightning: mode %d needs a list of chunks and their scratch", mode);
  ScanArgs a{q, k, v, q_stride, k_stride, v_stride, out, out_stride, state, decay, cu_q, state_slot, heads, dk, dv, act,
             (const int4*)items, scratch};
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) return launch_mode<float>(a, n_items, mode, s);
  if (dtype == LMSF_BF16) return launch_mode<bf16>(a, n_items, mode, s);
  LMSF_REFUSE("lightning: unknown dtype code %d", dtype);
}

// spans: int32 [n_spans][4] = (request, first chunk item, end chunk item, 0), one per long portion.
LMSF_API int lmsf_lightning_prefix(float* scratch, float* state, const float* decay, const int* state_slot, const int* items,
                                   const int* spans, int n_spans, int heads, int dk, int dv, void* stream) {
  using namespace lmsf;
  if (n_spans <= 0) return 0;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dv <= 0) LMSF_REFUSE("lightning: heads=%d dk=%d dv=%d", heads, dk, dv);
  const int per_head = dk * dv;
  dim3 grid(n_spans, heads, min(64, ceil_div(per_head, 256)));
  lightning_prefix_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(scratch, state, decay, state_slot, (const int4*)items,
                                                                   (const int4*)spans, heads, per_head);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_gated_norm(void* out, const float* x, long long x_stride, const void* gate, long long gate_stride,
                             const float* w, int n, int width, float eps, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (width <= 0 || !(eps > 0.f)) LMSF_REFUSE("gated_norm: width=%d, eps must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("gated_norm: unknown dtype code %d", dtype);
  const size_t el = dtype == LMSF_F32 ? 4 : 2;
  // four values per access where every row starts on a 16-byte (float32) or 8-byte (bfloat16) boundary
  const bool wide = width % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 && ((uintptr_t)x | (uintptr_t)w) % 16 == 0 &&
                    ((uintptr_t)gate | (uintptr_t)out) % (4 * el) == 0;
  if (dtype == LMSF_F32) {
    if (wide) gated_norm_kernel<float, 4><<<n, 256, 0, s>>>((float*)out, x, x_stride, (const float*)gate, gate_stride, w, width, eps);
    else gated_norm_kernel<float, 1><<<n, 256, 0, s>>>((float*)out, x, x_stride, (const float*)gate, gate_stride, w, width, eps);
  } else {
    if (wide) gated_norm_kernel<bf16, 4><<<n, 256, 0, s>>>((bf16*)out, x, x_stride, (const bf16*)gate, gate_stride, w, width, eps);
    else gated_norm_kernel<bf16, 1><<<n, 256, 0, s>>>((bf16*)out, x, x_stride, (const bf16*)gate, gate_stride, w, width, eps);
  }
  return LMSF_LAUNCH_STATUS();
}
