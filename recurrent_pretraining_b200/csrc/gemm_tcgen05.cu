// Persistent warp-specialised bf16 GEMM for sm_100a:  C[M,N] (+)= A[M,K] * B[N,K]^T  with fp32 accumulation in
// tensor memory.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled smem ring, mbarrier complete_tx)
//   warp 1      : MMA issuer    (one elected thread, tcgen05.mma 128 x BN x 16, tcgen05.commit frees smem stages)
//   warps 2..5  : epilogue      (tcgen05.ld from the *other* TMEM accumulator while the next tile is multiplied)
//
// One CTA per SM walks a static tile list (m fastest so that the CTAs in flight share B tiles through L2).
// Both operands may be K-major ([rows, K] row-major) or MN-major ([K, rows] row-major), which covers
// forward (x W^T), dgrad (dy W) and wgrad (dy^T x) without transposed copies.  Ragged M/N/K are handled by
// TMA zero fill on loads and by predicated stores.  An optional second A operand continues the K loop
// (y = x Ws^T + e We^T against one [N, K1+K2] weight): the recurrent adapter without a concatenation.
//
// Epilogues: bf16 store, fp32 store, fp32 accumulate (weight gradients summed over recurrences), bf16 store of
// acc + residual, and SwiGLU (B rows n and n + N are the gate and up rows; output silu(gate) * up).
#include <cuda.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace b200 {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row

template <int BN, int MODE>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;   // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int NB = is_swiglu(MODE) ? 2 : 1;  // SwiGLU stages a gate tile and an up tile
  static constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
  static constexpr int STAGES = (STAGE_BYTES > 32768) ? 4 : 6;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024 for manual alignment
};

template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
            const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using L = SmemLayout<BN, MODE>;
  constexpr int STAGES = L::STAGES;
  // accumulator width in TMEM columns: SwiGLU keeps gate and up side by side
  constexpr int ACC_COLS = is_swiglu(MODE) ? 2 * BN : BN;
  static_assert(ACC_COLS <= 256, "accumulator too wide");
  // two accumulators; tensor memory is allocated in powers of two >= 32 columns, and only as much as they need, so
  // that a dependent kernel launched early (programmatic dependent launch) can allocate beside a resident one
  constexpr int ACC_STRIDE = ACC_COLS <= 16 ? 16 : (ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : 256)));
  constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

  pdl_trigger();   // a dependent kernel may become resident beside this one; it waits for this grid before it reads
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int ksplit = p.ksplit > 1 ? p.ksplit : 1;
  const int num_tiles = tiles_m * tiles_n * ksplit;   // work items: (output tile, K range)
  const int nk1 = (p.K1 + BK - 1) / BK;
  const int nk2 = (p.K2 + BK - 1) / BK;
  const int nk = nk1 + nk2;
  // Work items of this CTA, by index: (output tile, k-block range).  Default: items blockIdx.x, +gridDim.x, ... of the
  // (tile, K range) list.  Stream-K: the CTA owns units [u0, u1) of the flattened (tile, k-block) space -- an equal
  // share for every CTA, whatever the tile count -- and its i-th item is the part of tile u0 / nk + i inside it.
  const long long sk_total = static_cast<long long>(tiles_m) * tiles_n * nk;
  const long long sk_u0 = sk_total * blockIdx.x / gridDim.x, sk_u1 = sk_total * (blockIdx.x + 1) / gridDim.x;
  const int sk_t0 = static_cast<int>(sk_u0 / nk);
  auto work_item = [&](int i, int& ot, int& kb0, int& kb1) -> bool {
    if (p.streamk) {
      ot = sk_t0 + i;
      const long long base = static_cast<long long>(ot) * nk;
      if (base >= sk_u1 || sk_u0 >= sk_u1) return false;
      kb0 = i == 0 ? static_cast<int>(sk_u0 - base) : 0;
      kb1 = sk_u1 - base < nk ? static_cast<int>(sk_u1 - base) : nk;
      return true;
    }
    const int tile = blockIdx.x + i * gridDim.x;
    if (tile >= num_tiles) return false;
    ot = tile / ksplit;
    const int ks = tile % ksplit;
    kb0 = static_cast<int>(static_cast<long long>(nk) * ks / ksplit);
    kb1 = static_cast<int>(static_cast<long long>(nk) * (ks + 1) / ksplit);
    return true;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above overlapped the predecessor's tail; operands and outputs are touched from here on.  With early_a
  // the A operand is constant data (decode weights): the producer thread starts streaming it before it waits for the
  // predecessor, which only produces the B operand.
  const bool early_thread = p.early_a && threadIdx.x == 0;
  if (!early_thread) pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (nk2 > 0) tma_prefetch_desc(&tmA2);
      uint32_t it = 0;
      bool ok = true;
      // phase 0 (early_a only): A tiles of the first STAGES k-blocks, before the wait for the predecessor;
      // phase 1: everything else (for those first k-blocks only the B tiles are left)
      for (int phase = early_thread ? 0 : 1; phase < 2 && ok; ++phase) {
        it = 0;
        int ot, kb0, kb1;
        bool more = true;
        for (int wi = 0; ok && more && work_item(wi, ot, kb0, kb1); ++wi) {
          int mt, nt;
          tile_coords(ot, tiles_m, tiles_n, p.raster, mt, nt);
          const int m0 = mt * BM, n0 = nt * BN;
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            if (phase == 0 && it >= STAGES) { more = false; break; }
            const bool a_done = early_thread && phase == 1 && it < STAGES;   // loaded in phase 0
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            uint8_t* sa = smem + s * L::STAGE_BYTES;
            uint8_t* sb = sa + L::A_BYTES;
            const bool second = kb >= nk1;
            const int ka = (second ? (kb - nk1) : kb) * BK;          // k offset inside the A operand
            const int kbcol = second ? (p.K1 + ka) : ka;             // k offset inside B
            if (!a_done) {
              if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_WAIT_STAGE_EMPTY)) { ok = false; break; }
              mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
              if constexpr (!A_MN) {
                if (second) tma_load_2d(sa, &tmA2, &full_bar[s], ka, m0);
                else tma_load_2d(sa, &tmA, &full_bar[s], ka, m0);
              } else {
#pragma unroll
                for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[s], m0 + c * 64, ka);
              }
            }
            if (phase == 0) continue;
            if constexpr (!B_MN) {
              tma_load_2d(sb, &tmB, &full_bar[s], kbcol, n0);
              if constexpr (is_swiglu(MODE)) tma_load_2d(sb + L::B_BYTES, &tmB, &full_bar[s], kbcol, n0 + p.swiglu_n);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[s], n0 + c * 64, kbcol);
            }
          }
        }
        if (phase == 0) pdl_wait();
      }
      // drain: every issued load must have landed before the CTA may exit
      const uint32_t issued = it;
      for (uint32_t j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j) {
        const int s = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(&full_bar[s], ph)) {
          if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      int ot, kb0, kb1;
      for (int wi = 0; ok && work_item(wi, ot, kb0, kb1); ++wi, ++tcount) {
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, ERR_WAIT_TMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 elements = 32 bytes inside the swizzle row.  MN-major: 16 k-rows of 128 bytes.
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, IDESC, (kb > kb0 || k) ? 1u : 0u);
            if constexpr (is_swiglu(MODE)) {
              const uint64_t b2 = make_smem_desc(sb + L::B_BYTES + k * 32, 16, 1024);
              umma_bf16(d_tmem + BN, adesc, b2, IDESC, (kb > kb0 || k) ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[s]);  // smem stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t tcount = 0;
    int ot, kb0, kb1;
    for (int wi = 0; work_item(wi, ot, kb0, kb1); ++wi, ++tcount) {
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      int mt, nt;
      tile_coords(ot, tiles_m, tiles_n, p.raster, mt, nt);
      const int m0 = mt * BM, n0 = nt * BN;
      if (!mbar_wait(&tfull_bar[acc], aph, abort_flag, p.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_STRIDE + (static_cast<uint32_t>(quad * 32) << 16);
      epilogue_tile<BN, MODE>(p, taddr, m0 + quad * 32 + lane, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements); the box is
// [box_rows, 64 columns] with 128-byte swizzle.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 2-D fp32 tensor map over a row-major [rows, cols] matrix (leading dimension ld elements) for bulk stores / reductions
// of [box_rows, 32 columns] boxes staged with 128-byte swizzle.
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 4) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN, int MODE>
static int launch(const CUtensorMap& ta, const CUtensorMap& ta2, const CUtensorMap& tb, const GemmParams& p,
                  cudaStream_t stream, int max_ctas) {
  using L = SmemLayout<BN, MODE>;
  constexpr int SMEM = L::TOTAL;
  static_assert(!is_swiglu(MODE) || BN == 128, "SwiGLU epilogue uses BN = 128");
  auto kern = gemm_kernel<BN, A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * (p.ksplit > 1 ? p.ksplit : 1);
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (p.streamk) {  // one CTA per SM as long as each gets at least four k-blocks
    const long long units = static_cast<long long>(tiles) * ((p.K1 + BK - 1) / BK + (p.K2 + BK - 1) / BK);
    grid = units / 4 < num_sms() ? static_cast<int>(units / 4 > 0 ? units / 4 : 1) : num_sms();
  }
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;
  if (launch_k(kern, dim3(grid), dim3(192), SMEM, stream, ta, ta2, tb, p) != cudaSuccess) return -11;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace b200

static int g_raster = 8;   // m tiles per raster group of the large GEMMs (0: m fastest)
B200_API int b200_gemm_set_raster(int group) { const int old = g_raster; g_raster = group < 0 ? 0 : group; return old; }

int g_b200_pdl = 0;
extern "C" __attribute__((visibility("default"))) int b200_set_pdl(int on) {
  const int old = g_b200_pdl;
  g_b200_pdl = on ? 1 : 0;
  return old;
}

namespace b200 {
int gemm_2cta_dispatch(const void* A, const void* A2, const void* B, const GemmParams& p, int lda, int lda2, int ldb,
                       int a_mn, int b_mn, int out_mode, int bn, int max_ctas, cudaStream_t st);
static int g_use_2cta = 1;
}  // namespace b200

using namespace b200;

// 1: prefer the 2-CTA (cta_group::2) kernel where it applies (default); 0: always the 1-CTA kernel.
B200_API int b200_gemm_set_2cta(int enable) {
  const int old = g_use_2cta;
  g_use_2cta = enable;
  return old;
}

// C[M,N] (+)= A * B^T.
//   a_mn = 0: A is [M, K1] row-major (lda);  a_mn = 1: A is [K1, M] row-major (lda)
//   b_mn = 0: B is [N, K]  row-major (ldb);  b_mn = 1: B is [K, N]  row-major (ldb),  K = K1 + K2
//   A2 (optional, K-major only): second A operand [M, K2] multiplied against B columns K1..K1+K2
//   out_mode: see OutMode.  For OUT_SWIGLU, N is the output width I and B holds 2I rows ([gate; up]).
//   bn: tile width (256, 240 or 128); 0 picks one.  max_ctas > 0 caps the grid (used to leave SMs to a
//   concurrent communication kernel).
// Arguments of the next OUT_BF16_ROPE call (host-side state of the calling thread; set right before b200_gemm).
struct RopeArgs { const float* cos; const float* sin; const float* bias; int S, D, width; };
static thread_local RopeArgs g_rope = {nullptr, nullptr, nullptr, 0, 0, 0};
B200_API void b200_gemm_set_rope(const float* cos, const float* sin, const float* bias, int S, int D, int width) {
  g_rope = {cos, sin, bias, S, D, width};
}

// Arguments of the next OUT_BF16_LSE call (same convention as b200_gemm_set_rope).
struct LseArgs { void* part; float* tgt; const long long* labels; float scale; };
static thread_local LseArgs g_lse = {nullptr, nullptr, nullptr, 1.f};
B200_API void b200_gemm_set_lse(void* part, float* tgt, const long long* labels, float scale) {
  g_lse = {part, tgt, labels, scale};
}

B200_API int b200_gemm(const void* A, const void* A2, const void* B, void* C, const void* resid, int M, int N,
                       int K1, int K2, int lda, int lda2, int ldb, int ldc, int ld_resid, int a_mn, int b_mn,
                       int out_mode, int bn, int max_ctas, void* stream, int* err) {
  if (M <= 0 || N <= 0 || K1 <= 0) return 0;
  if (K2 > 0 && (a_mn || b_mn || (K1 & 7))) return -20;
  const int K = K1 + K2;
  if (bn == 0) {
    if (is_swiglu(out_mode)) bn = 128;
    else if (b_mn) bn = (N <= 128) ? 128 : 256;
    else if (N <= 128) bn = 128;
    else bn = (!a_mn && N % 256 != 0 && N % 240 == 0) ? 240 : 256;   // 240-wide tiles exist for the NT layout only
  }
  if (b_mn && bn == 240) return -21;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  GemmParams p = {};
  p.M = M; p.N = N; p.K1 = K1; p.K2 = K2; p.ldc = ldc; p.ld_resid = ld_resid; p.swiglu_n = N; p.ksplit = 1;
  p.C = C; p.resid = reinterpret_cast<const __nv_bfloat16*>(resid); p.err = err;
  // a very long contraction (the head's input gradient, K = vocabulary) keeps the m-fastest order: every wave then
  // shares each B k-slice among all 16 m tiles at once (measured 1173 vs 998 TFLOP/s with groups of 8)
  p.raster = (K1 + K2 >= 32768) ? 0 : g_raster;
  p.rope_cos = g_rope.cos; p.rope_sin = g_rope.sin; p.rope_bias = g_rope.bias;
  p.rope_S = g_rope.S; p.rope_D = g_rope.D; p.rope_width = g_rope.width;
  p.lse_part = reinterpret_cast<float4*>(g_lse.part); p.lse_tgt = g_lse.tgt; p.lse_labels = g_lse.labels;
  p.lse_scale = g_lse.scale;
  if (out_mode == OUT_BF16_LSE && (!p.lse_part || !p.lse_tgt || !p.lse_labels || a_mn || b_mn || bn != 256)) return -27;
  if (out_mode == OUT_BF16_ROPE && (!p.rope_cos || p.rope_D <= 0 || (p.rope_D & 1) || (p.rope_width & 1))) return -25;
  if (g_use_2cta && M >= 256 && (bn == 256 || bn == 240 || (is_swiglu(out_mode) && !a_mn && !b_mn))) {
    // SwiGLU on the pair kernel: a 256-wide MMA tile = 128 gate columns (CTA 0's half of B) + 128 up columns (CTA 1's)
    const int bn2 = is_swiglu(out_mode) ? 256 : bn;
    const int rc2 = gemm_2cta_dispatch(A, A2, B, p, lda, lda2, ldb, a_mn, b_mn, out_mode, bn2, max_ctas, st);
    if (rc2 != -100) return rc2;
  }
  CUtensorMap ta, ta2, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d_bf16(&ta, A, M, K1, lda, BM, BK);
  else rc = make_tmap_2d_bf16(&ta, A, K1, M, lda, BK, 64);
  if (rc) return rc;
  ta2 = ta;
  if (K2 > 0) {
    rc = make_tmap_2d_bf16(&ta2, A2, M, K2, lda2, BM, BK);
    if (rc) return rc;
  }
  const int brows = is_swiglu(out_mode) ? 2 * N : N;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, brows, K, ldb, bn, BK);
  else rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, 64);
  if (rc) return rc;

#define DISPATCH_MODE(BN_, AMN_, BMN_)                                                            \
  switch (out_mode) {                                                                             \
    case OUT_BF16: return launch<BN_, AMN_, BMN_, OUT_BF16>(ta, ta2, tb, p, st, max_ctas);        \
    case OUT_F32: return launch<BN_, AMN_, BMN_, OUT_F32>(ta, ta2, tb, p, st, max_ctas);          \
    case OUT_F32_ACC: return launch<BN_, AMN_, BMN_, OUT_F32_ACC>(ta, ta2, tb, p, st, max_ctas);  \
    case OUT_BF16_RESID: return launch<BN_, AMN_, BMN_, OUT_BF16_RESID>(ta, ta2, tb, p, st, max_ctas); \
    default: return -22;                                                                          \
  }

  if (out_mode == OUT_SWIGLU) {
    if (a_mn || b_mn || bn != 128) return -23;
    return launch<128, false, false, OUT_SWIGLU>(ta, ta2, tb, p, st, max_ctas);
  }
  if (out_mode == OUT_BF16_LSE) return launch<256, false, false, OUT_BF16_LSE>(ta, ta2, tb, p, st, max_ctas);
  if (out_mode == OUT_SWIGLU_SAVE) {
    if (a_mn || b_mn || bn != 128 || !resid) return -23;
    return launch<128, false, false, OUT_SWIGLU_SAVE>(ta, ta2, tb, p, st, max_ctas);
  }
  if (out_mode == OUT_DSWIGLU) {
    if (a_mn || !b_mn || !resid) return -26;
    if (bn == 128) return launch<128, false, true, OUT_DSWIGLU>(ta, ta2, tb, p, st, max_ctas);
    return launch<256, false, true, OUT_DSWIGLU>(ta, ta2, tb, p, st, max_ctas);
  }
  if (out_mode == OUT_BF16_ROPE) {
    if (a_mn || b_mn) return -24;
    if (bn == 240) return launch<240, false, false, OUT_BF16_ROPE>(ta, ta2, tb, p, st, max_ctas);
    if (bn == 128) return launch<128, false, false, OUT_BF16_ROPE>(ta, ta2, tb, p, st, max_ctas);
    return launch<256, false, false, OUT_BF16_ROPE>(ta, ta2, tb, p, st, max_ctas);
  }
  if (!a_mn && !b_mn) {
    if (bn == 256) { DISPATCH_MODE(256, false, false) }
    if (bn == 240) { DISPATCH_MODE(240, false, false) }
    if (bn == 128) { DISPATCH_MODE(128, false, false) }
  } else if (!a_mn && b_mn) {
    if (bn == 256) { DISPATCH_MODE(256, false, true) }
    if (bn == 128) { DISPATCH_MODE(128, false, true) }
  } else if (a_mn && b_mn) {
    if (bn == 256) { DISPATCH_MODE(256, true, true) }
    if (bn == 128) { DISPATCH_MODE(128, true, true) }
  } else {
    if (bn == 256) { DISPATCH_MODE(256, true, false) }
    if (bn == 128) { DISPATCH_MODE(128, true, false) }
  }
#undef DISPATCH_MODE
  return -24;
}


static int g_skinny_streamk = 1;
B200_API int b200_skinny_set_streamk(int on) { const int old = g_skinny_streamk; g_skinny_streamk = on; return old; }

// Skinny (decode) GEMM:  out[Bt, N] = x[Bt, K] * W[N, K]^T  for Bt <= 64, computed as W * x^T so that the streamed
// weight rows fill the 128-row MMA dimension and every SM pulls its own slice of W.  When N/128 tiles cannot occupy
// the machine the K range is split and partial sums are accumulated with fp32 atomics into `work` ([Bt, N] fp32,
// zeroed here when zero_work != 0); the caller then consumes `work` (b200_cast_zero / b200_add_rmsnorm_f32).  Returns 1 if `work` holds the result, 0 if
// `out` does, negative on error.
B200_API int b200_gemm_skinny(const void* x, const void* W, void* out, float* work, int Bt, int N, int K, int ldx,
                              int ldw, int ldo, int zero_work, void* stream, int* err) {
  if (Bt <= 0 || Bt > 64 || N <= 0 || K <= 0) return -30;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int bn = Bt <= 16 ? 16 : (Bt <= 32 ? 32 : 64);
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, W, N, K, ldw, BM, BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, x, Bt, K, ldx, bn, BK);
  if (rc) return rc;
  const int tiles = (N + BM - 1) / BM;
  const int nk = (K + BK - 1) / BK;
  // Fewer weight-row tiles than SMs: stream-K.  A fixed K split leaves tiles * ksplit work items, which rarely divide
  // by the SM count (N = 5280: 42 tiles * 4 = 168 items on 148 SMs ran as two waves, 57 % of the machine); with
  // stream-K every SM streams the same number of weight bytes.
  // More tiles than SMs but not a multiple of them (gate-up: 280 tiles = 1.89 waves) gains too, as long as the batch is
  // narrow: the accumulation costs 128 x Bt atomics per (tile, CTA) piece.
  const bool streamk = work && nk >= 8 && g_skinny_streamk &&
                       (tiles < num_sms() || (Bt <= 16 && tiles % num_sms() != 0));
  GemmParams p = {};
  p.M = N; p.N = Bt; p.K1 = K; p.K2 = 0; p.ld_resid = 0; p.swiglu_n = 0; p.resid = nullptr; p.err = err;
  p.ksplit = 1;
  p.streamk = streamk ? 1 : 0;
  p.early_a = 1;   // W is constant between launches: stream it while the predecessor (which produces x) still runs
  if (streamk) {
    // zero_work = 0: the caller guarantees `work` is already zero (its consumer kernels clear it after reading)
    if (zero_work && cudaMemsetAsync(work, 0, static_cast<size_t>(Bt) * N * sizeof(float), st) != cudaSuccess)
      return -31;
    p.C = work; p.ldc = N;
    switch (bn) {
      case 16: rc = launch<16, false, false, OUT_F32_T_ATOMIC>(ta, ta, tb, p, st, 0); break;
      case 32: rc = launch<32, false, false, OUT_F32_T_ATOMIC>(ta, ta, tb, p, st, 0); break;
      default: rc = launch<64, false, false, OUT_F32_T_ATOMIC>(ta, ta, tb, p, st, 0); break;
    }
    return rc ? rc : 1;
  }
  p.C = out; p.ldc = ldo;
  switch (bn) {
    case 16: return launch<16, false, false, OUT_BF16_T>(ta, ta, tb, p, st, 0);
    case 32: return launch<32, false, false, OUT_BF16_T>(ta, ta, tb, p, st, 0);
    default: return launch<64, false, false, OUT_BF16_T>(ta, ta, tb, p, st, 0);
  }
}
