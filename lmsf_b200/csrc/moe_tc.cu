// The experts' products on the 5th-generation tensor cores (bfloat16): one launch for all experts.
//
// A block computes one tile: 128 rows of one expert (rows of the sorted (token, choice) list, see moe.cu) times 256
// output features of that expert's matrix, C = act(A W_e^T).  K is walked in steps of 64 through a ring of kStages
// shared-memory stages; a stage holds a [128 x 64] slab of A and a [256 x 64] slab of W_e, each row 128 bytes, 16-byte
// chunk c of row r at chunk c ^ (r & 7) (the 128-byte swizzle that the matrix descriptors name).
//   warps 0-3  bring the slab of A with cp.async: its rows are GATHERED through the pair list (the up projection
//              reads each token's activation row where it lies; no copy sorted by expert is made), rows beyond the
//              tile's and columns beyond K are zero-filled.  Thread 0 also asks the copy engine for the slab of W_e: two
//              boxes of 128 rows of the experts' matrices seen as one [experts x N, K] tensor (rows past this expert's
//              are another expert's or zeros; their columns of the result are not stored).  Afterwards the same warps
//              are the epilogue: each thread reads its row of the accumulator from tensor memory, applies the activation
//              and stores it
//   warp 4     issues tcgen05.mma (M 128, N 256, K 16, float32 accumulator in 256 columns of tensor memory) from one
//              elected lane, frees a stage with tcgen05.commit, and signals the epilogue after the last step
// Every wait is bounded; a block that gives up raises error code 4 and leaves its tile unwritten.
#include "tc_common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_moe_tc)

namespace lmsf {

using namespace tc;

constexpr int TM = 128, TN = 256, TK = 64;
constexpr int kStages = 4;
constexpr int kSlab = TM * TK * 2;                 // 16 KB: the slab of A, and each of the two boxes of W
constexpr int kWBytes = TN * TK * 2;               // 32 KB
constexpr int kStageBytes = kSlab + kWBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024;
constexpr uint32_t kTmemCols = 256;
constexpr int kLoaders = 128;

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct GroupedArgs {
  void* C; const bf16* A; const bf16* W;
  const int* gather; const int* tiles; const int* meta;
  int N, K; long long lda, ldc;
  int* error_flag;
};

template <int ACT, typename TC>
__global__ void __launch_bounds__(160) moe_grouped_tc_kernel(const GroupedArgs a, const __grid_constant__ CUtensorMap w_map) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kStages + 1];
  __shared__ uint32_t tmem_base_mem;
  __shared__ int failed_mem;
  __shared__ int src_row[TM];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int tile = blockIdx.y;
  if (tile >= a.meta[0]) return;
  const int e = a.tiles[4 * tile], row0 = a.tiles[4 * tile + 1], rows = a.tiles[4 * tile + 2];
  const int n0 = blockIdx.x * TN;
  const uint32_t smem = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  const uint32_t acc_full = bar0 + 8u * (2 * kStages);
  volatile int* failed = &failed_mem;
  if (tid == 0) {
    // a stage is full after every loader's cp.async have landed and the copy engine's bytes have arrived
    for (int s = 0; s < kStages; ++s) { mbar_init(full(s), kLoaders + 1); mbar_init(empty(s), 1); }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    failed_mem = 0;
  }
  if (tid < TM) src_row[tid] = tid < rows ? (a.gather ? a.gather[row0 + tid] : row0 + tid) : -1;
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_mem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_mem;
  const int k_steps = (a.K + TK - 1) / TK;

  if (warp < 4) {
    // ---------------------------------------------------------------- the slabs: thread t brings chunk t % 8 of rows t / 8 + 16 i
    const int c = tid & 7, r_base = tid >> 3;
    const int w_row = e * a.N + n0;                   // first row of the slab of W in the [experts x N, K] tensor
    bool ok = true;
    for (int ks = 0; ks < k_steps && ok; ++ks) {
      const int s = ks % kStages;
      if (ks >= kStages && !mbar_wait_f(empty(s), (uint32_t)((ks / kStages - 1) & 1), failed)) { ok = false; break; }
      const uint32_t sa = smem + s * kStageBytes, sw = sa + kSlab;
      if (tid == 0) {
        mbar_arrive_expect_tx(full(s), kWBytes);
        tma_load_box_2d(sw, &w_map, ks * TK, w_row, full(s));
        tma_load_box_2d(sw + kSlab, &w_map, ks * TK, w_row + TM, full(s));
      }
      const int k = ks * TK + c * 8;
      const bool k_ok = k < a.K;
#pragma unroll
      for (int i = 0; i < TM / 16; ++i) {
        const int r = r_base + 16 * i;
        const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
        const int ar = src_row[r];
        const bool a_ok = k_ok && ar >= 0;
        cp16(sa + off, a_ok ? (const void*)(a.A + (size_t)ar * a.lda + k) : (const void*)a.A, a_ok ? 16 : 0);
      }
      cp_async_arrive(full(s));
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");      // no copy of this block is in flight when it ends
    // (the copy engine's boxes are waited for by the issuing warp before every product; if that warp gave up, the
    // barriers of the boxes still in flight are drained here)
    if (*failed && tid == 0)
      for (int g = max(0, k_steps - kStages); g < k_steps; ++g) mbar_wait_drain(full(g % kStages), (uint32_t)((g / kStages) & 1));
    // ---------------------------------------------------------------- the epilogue: thread t holds row t of the accumulator
    if (ok && mbar_wait_f(acc_full, 0, failed)) {
      tc_fence_after();
      const int r = tid;
      TC* crow = (TC*)a.C + (size_t)(row0 + r) * a.ldc;
#pragma unroll
      for (int cb = 0; cb < TN / 32; ++cb) {
        float v[32];
        tmem_ld32_issue(tmem + ((uint32_t)(warp * 32) << 16) + cb * 32, v);
        tmem_wait_ld();
        if (r < rows) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (ACT == 1) { v[j] = fmaxf(v[j], 0.f); v[j] *= v[j]; }
          const int nb = n0 + cb * 32;
          if (nb + 32 <= a.N && a.ldc % 8 == 0 && (uintptr_t)a.C % 16 == 0) {      // whole 16-byte words
            if (sizeof(TC) == 2) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 w;
                w.x = pack2(v[j], v[j + 1]); w.y = pack2(v[j + 2], v[j + 3]); w.z = pack2(v[j + 4], v[j + 5]); w.w = pack2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(crow + nb + j) = w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(crow + nb + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < a.N) crow[nb + j] = from_f32<TC>(v[j]);
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- tensor-core issue
    constexpr uint32_t idesc = instr_desc(TM, TN, 0);
    const bool leader = elect_one();
    bool ok = true;
    for (int ks = 0; ks < k_steps; ++ks) {
      const int s = ks % kStages;
      if (!mbar_wait_f(full(s), (uint32_t)((ks / kStages) & 1), failed)) { ok = false; break; }
      fence_async_smem();
      tc_fence_after();
      const uint64_t da = smem_desc(smem + s * kStageBytes, 16, 1024), dw = smem_desc(smem + s * kStageBytes + kSlab, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < TK / 16; ++kk)
        umma(leader, tmem, da + (uint64_t)((kk * 32) >> 4), dw + (uint64_t)((kk * 32) >> 4), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
      umma_commit(leader, empty(s));
    }
    if (ok) umma_commit(leader, acc_full);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*failed && tid == 0 && a.error_flag) atomicExch(a.error_flag, 4);
  if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

template <int ACT, typename TC>
static int launch(const GroupedArgs& a, const CUtensorMap& w_map, int max_tiles, cudaStream_t s) {
  auto kernel = moe_grouped_tc_kernel<ACT, TC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(ceil_div(a.N, TN), max_tiles);
  kernel<<<grid, 160, kSmemBytes, s>>>(a, w_map);
  return LMSF_LAUNCH_STATUS();
}

// The experts' matrices as one 2-d tensor for the copy engine: (K, experts x N), a box of 64 x 128, written 128-byte
// swizzled.  Made once per (address, geometry).
static const CUtensorMap* weight_map(const void* W, long long rows, int K, const char** why) {
  using Key = std::tuple<const void*, long long, int>;
  static std::map<Key, CUtensorMap> maps;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{W, rows, K};
  auto it = maps.find(key);
  if (it != maps.end()) return &it->second;
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) { *why = "the driver has no cuTensorMapEncodeTiled"; return nullptr; }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)TM};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(W), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled refused the experts' geometry"; return nullptr; }
  return &maps.emplace(key, m).first->second;
}

}  // namespace lmsf

LMSF_API int lmsf_moe_tc_tile_rows() { return lmsf::TM; }

// C: [pairs, N] bfloat16 (out_dtype 1) or float32 (0); A: bfloat16 rows of K values; W: bfloat16 [experts, N, K];
// tiles of 128 rows (moe_align with tile_rows = 128); act: 0 none, 1 relu squared.
LMSF_API int lmsf_moe_grouped_tc(void* C, const void* A, const void* W, const int* gather, const int* tiles, const int* meta,
                                 int max_tiles, int experts, int N, int K, long long lda, long long ldc, int act, int out_dtype,
                                 int* error_flag, void* stream) {
  using namespace lmsf;
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || lda < K || ldc < N || ((uintptr_t)A | (uintptr_t)W) % 16)
    LMSF_REFUSE("moe_tc: K=%d lda=%lld must be multiples of 8 and the operands 16-byte aligned", K, lda);
  if (max_tiles > 65535) LMSF_REFUSE("moe_tc: more than 65535 row tiles in one launch");
  if (act != 0 && act != 1) LMSF_REFUSE("moe_tc: unknown activation code %d", act);
  if (experts <= 0) LMSF_REFUSE("moe_tc: experts=%d", experts);
  const char* why = "";
  const CUtensorMap* wm = weight_map(W, (long long)experts * N, K, &why);
  if (!wm) LMSF_REFUSE("moe_tc: %s", why);
  GroupedArgs a{C, (const bf16*)A, (const bf16*)W, gather, tiles, meta, N, K, lda, ldc, error_flag};
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == LMSF_BF16) return act ? launch<1, bf16>(a, *wm, max_tiles, s) : launch<0, bf16>(a, *wm, max_tiles, s);
  if (out_dtype == LMSF_F32) return act ? launch<1, float>(a, *wm, max_tiles, s) : launch<0, float>(a, *wm, max_tiles, s);
  LMSF_REFUSE("moe_tc: unknown dtype code %d", out_dtype);
}
