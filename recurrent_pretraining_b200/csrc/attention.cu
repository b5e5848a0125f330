// Causal flash attention for sm_100a on a packed, already rotated qkv tensor [B, S, (H + 2 Hkv) * D], D <= 128,
// D % 16 == 0 (the flagship uses D = 96).  tcgen05 MMAs with the score tile S and the partial output in
// tensor memory, operands staged by TMA into 128-byte-swizzled shared memory.
//
// Forward, one CTA per (128-query block, head, batch):
//   warp 0     TMA producer: Q once, then K_j / V_j (128 keys) through a 2-stage ring
//   warp 1     MMA issuer:   S_j = Q K_j^T  (into one of two TMEM score buffers, issued one block ahead),
//                            O_j = P_j V_j  (fresh partial product, V read MN-major)
//   warps 2-5  softmax:      one query row per thread; two passes over the TMEM score row (max, then exp2 / sum /
//                            bf16 P written to swizzled smem); partial outputs are folded into fp32 registers with
//                            the usual online-softmax rescale, so TMEM never needs a read-modify-write
// Output: o [B, S, H*D] bf16 and the natural-log row log-sum-exp lse [B, H, S] fp32 (used by the backward).
//
// Backward, one CTA per (128-key block, kv-head... query head, batch), looping over the query blocks at or below
// the diagonal: S and dP = dO V^T are recomputed into TMEM, P and dS are written once to smem and used both as a
// K-major operand (dQ = dS K) and as an MN-major operand (dV += P^T dO, dK += dS^T Q); dK/dV accumulate in TMEM
// over the whole loop, dQ tiles are added to an fp32 buffer with vector atomics and converted afterwards.
#include <cuda.h>

#include "common.cuh"

namespace b200 {

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D bf16 tensor map {d0 (contiguous), d1, d2} with byte strides for d1 and d2; box {box0, box1, 1}, 128B swizzle.
static int make_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                        CUtensorMapDataType dtype);
static int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
  return make_tmap_3d(out, base, d0, d1, d2, stride1_bytes, stride2_bytes, box0, box1,
                      CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
}
// 3-D tensor map {d0 (contiguous), d1, d2}; box {box0, box1, 1}; 128-byte swizzle (box0 * element size must be 128).
static int make_tmap_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                        CUtensorMapDataType dtype) {
  static EncodeTiledFn3 enc = nullptr;
  if (!enc) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -1;
    enc = reinterpret_cast<EncodeTiledFn3>(ptr);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

constexpr int ATT_BM = 128;  // queries per CTA
constexpr int ATT_BN = 128;  // keys per step
constexpr int PANEL_BYTES = 128 * 128;  // 128 rows x 128 bytes (64 bf16)

struct AttnParams {
  int B, S, H, Hkv, D;
  int wq, wk;          // widths of the q and k sections of a packed row
  float scale_log2;    // softmax scale * log2(e)
  __nv_bfloat16* o;    // [B, S, H*D]
  float* lse;          // [B, H, S]
  int* err;
};

struct FwdBars {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_ready, o_full, o_empty;
  uint32_t tmem_slot;
  int abort_flag;
};

template <int D>
__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  constexpr int KSTEPS = D / 16;
  constexpr uint32_t IDESC_S = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(ATT_BM, D, 0, 1);
  constexpr int TILE_BYTES = 2 * PANEL_BYTES;  // two 64-wide panels (the second is partly unused for D < 128)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;        // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;    // 2 stages
  uint8_t* sP = sV + 2 * TILE_BYTES;
  FwdBars* bars = reinterpret_cast<FwdBars*>(sP + TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + ATT_BM - 1) / ATT_BM;
  const int qb = nqb - 1 - blockIdx.x;  // heavy (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * ATT_BM;
  const int nkb = min(qb + 1, (p.S + ATT_BN - 1) / ATT_BN);
  const int xq = h * D, xk = p.wq + hk * D, xv = p.wq + p.wk + hk * D;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4);
    }
    mbar_init(&bars->p_ready, 4);
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->o_empty, 4);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm);
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      tma_load_3d(sQ, &tm, &bars->q_full, xq, q0, b);
      tma_load_3d(sQ + PANEL_BYTES, &tm, &bars->q_full, xq + 64, q0, b);
      int issued = 0;
      for (int j = 0; j < nkb; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, &tm, &bars->k_full[s], xk, j * ATT_BN, b);
        tma_load_3d(sK + s * TILE_BYTES + PANEL_BYTES, &tm, &bars->k_full[s], xk + 64, j * ATT_BN, b);
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_3d(sV + s * TILE_BYTES, &tm, &bars->v_full[s], xv, j * ATT_BN, b);
        tma_load_3d(sV + s * TILE_BYTES + PANEL_BYTES, &tm, &bars->v_full[s], xv + 64, j * ATT_BN, b);
        issued = j + 1;
      }
      // all issued loads must land before the CTA exits
      unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->q_full, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      for (int j = max(0, issued - 2); j < issued; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->k_full[s], ph) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
        while (!mbar_try_wait(&bars->v_full[s], ph) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t kb = aK + s * TILE_BYTES;
#pragma unroll
        for (int t = 0; t < KSTEPS; ++t) {
          const uint32_t off = (t >> 2) * PANEL_BYTES + (t & 3) * 32;
          umma_bf16(tmem_base + s * 128, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(kb + off, 16, 1024),
                    IDESC_S, t ? 1u : 0u);
        }
        umma_commit(&bars->s_full[s]);
      };
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.err, ERR_WAIT_ATTN) &&
                mbar_wait(&bars->k_full[0], 0, abort_flag, p.err, ERR_WAIT_ATTN);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < nkb && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nkb) {
          const int s1 = (j + 1) & 1;
          const uint32_t ph1 = ((j + 1) >> 1) & 1;
          if (!mbar_wait(&bars->k_full[s1], ph1, abort_flag, p.err, ERR_WAIT_ATTN) ||
              !mbar_wait(&bars->s_empty[s1], ph1 ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(&bars->p_ready, j & 1, abort_flag, p.err, ERR_WAIT_ATTN) ||
            !mbar_wait(&bars->v_full[s], ph, abort_flag, p.err, ERR_WAIT_ATTN) ||
            !mbar_wait(&bars->o_empty, (j & 1) ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
        tc_fence_after();
        const uint32_t vb = aV + s * TILE_BYTES;
#pragma unroll
        for (int t = 0; t < ATT_BN / 16; ++t) {
          const uint64_t adesc = make_smem_desc(aP + (t >> 2) * PANEL_BYTES + (t & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(vb + t * 2048, PANEL_BYTES, 1024);
          umma_bf16(tmem_o, adesc, bdesc, IDESC_O, t ? 1u : 0u);
        }
        umma_commit(&bars->o_full);
        umma_commit(&bars->kv_empty[s]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // query row inside the tile
    const int qrow = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&bars->s_full[s], ph, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + s * 128 + lane_addr;
      const bool diag = (j == qb);
      const int kbase = j * ATT_BN;
      // pass 1: row max
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < ATT_BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(ts + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t = __uint_as_float(v[i]) * p.scale_log2;
          if (diag && (kbase + c + i > qrow)) t = -INFINITY;
          mx = fmaxf(mx, t);
        }
      }
      const float m_new = mx;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      // fold the previous partial output (scaled by the previous alpha) before P is overwritten
      if (j > 0) {
        if (!mbar_wait(&bars->o_full, (j - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          uint32_t v[16];
          tmem_ld_32x16(tmem_o + lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[c + i] = acc[c + i] * alpha_prev + __uint_as_float(v[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->o_empty);
      }
      // pass 2: probabilities
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < ATT_BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(ts + c, v);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float t0 = __uint_as_float(v[i]) * p.scale_log2, t1 = __uint_as_float(v[i + 1]) * p.scale_log2;
          if (diag) {
            if (kbase + c + i > qrow) t0 = -INFINITY;
            if (kbase + c + i + 1 > qrow) t1 = -INFINITY;
          }
          const float p0 = (m_new == -INFINITY) ? 0.f : exp2f(t0 - m_new);
          const float p1 = (m_new == -INFINITY) ? 0.f : exp2f(t1 - m_new);
          packed[i >> 1] = pack_bf16x2(p0, p1);
          // sum what the tensor core will actually see
          const float2 pr = unpack_bf16x2(packed[i >> 1]);
          rowsum += pr.x + pr.y;
        }
        // keys [c, c+32) of this row: panel c/64, 16-byte chunks (c%64)/8 .. +3, XOR-swizzled with r%8
        uint8_t* prow = sP + (c >> 6) * PANEL_BYTES + r * 128;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int phys = (chunk0 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + phys * 16) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      tc_fence_before();
      l = l * alpha + rowsum;
      m = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->s_empty[s]);
        mbar_arrive(&bars->p_ready);
      }
    }
    // NOTE on alpha bookkeeping: acc holds sum_{i<j} O_i rescaled to max m_{j-1}; the partial O_{j-1} was
    // computed against m_{j-1}; when block j raises the max, both are multiplied by alpha_j on the next fold.
    if (ok && nkb > 0) {
      if (mbar_wait(&bars->o_full, (nkb - 1) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) {
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.o + (static_cast<size_t>(b) * p.S + qrow) * (p.H * D) + h * D;
#pragma unroll
        for (int c = 0; c < D; c += 16) {
          uint32_t v[16];
          tmem_ld_32x16(tmem_o + lane_addr + c, v);
          tmem_ld_wait();
          if (qrow < p.S) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2)
              o[i >> 1] = pack_bf16x2((acc[c + i] * alpha_prev + __uint_as_float(v[i])) * inv_l,
                                      (acc[c + i + 1] * alpha_prev + __uint_as_float(v[i + 1])) * inv_l);
            *reinterpret_cast<uint4*>(orow + c) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        if (qrow < p.S && p.lse)
          p.lse[(static_cast<size_t>(b) * p.H + h) * p.S + qrow] = (m + log2f(l)) * 0.6931471805599453f;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ------------------------------------------------------------------------------------------------ forward, v2
// Two 128-query tiles (A = even query block 2i, B = odd block 2i+1) per CTA with one softmax warpgroup each, so the
// tensor pipe works on one tile while the other tile's softmax runs:
//   warp 8      TMA: Q_A, Q_B once; K_j / V_j through a 2-stage ring (shared by both tiles)
//   warps 9-10  MMA (one issuing thread per tile): S_X = Q_X K_j^T into TMEM; O_X += P_X V_j with P_X read from TMEM (bf16, written over the first
//               half of S_X's columns by the softmax warps) and accumulated in TMEM across all key blocks
//   warps 0-3   softmax of tile A, warps 4-7 softmax of tile B: one row per thread, whole 128-column score row in
//               registers, single pass; the running max is only raised (and O rescaled in TMEM) when it grew by more
//               than 2^8, otherwise the stale max is kept -- P then stays below 256 and the final 1/l fixes the scale
// TMEM columns: S_A [0,128)  S_B [128,256)  O_A [256,256+D)  O_B [384,384+D).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe (no MUFU): floor by the 1.5 * 2^23 trick with round-down, cubic for the fractional part, the
// integer part added into the exponent field.  Relative error about 1e-4, below bf16 resolution.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.f);
  float t;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(t) : "f"(x), "f"(12582912.f));
  const float f = x - (t - 12582912.f);
  float pl = fmaf(f, 0.077119089663028717f, 0.227564394474029541f);
  pl = fmaf(pl, f, 0.695146143436431885f);
  pl = fmaf(pl, f, 1.f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(t) << 23));
}

// three-input max and packed two-wide fp32 arithmetic (sm_100): half the issue slots of the scalar forms
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n"
      "  .reg .b64 ra, rb, rc, rd;\n"
      "  mov.b64 ra, {%2, %3};\n"
      "  mov.b64 rb, {%4, %5};\n"
      "  mov.b64 rc, {%6, %7};\n"
      "  fma.rn.f32x2 rd, ra, rb, rc;\n"
      "  mov.b64 {%0, %1}, rd;\n"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n"
      "  .reg .b64 ra, rb, rd;\n"
      "  mov.b64 ra, {%2, %3};\n"
      "  mov.b64 rb, {%4, %5};\n"
      "  add.rn.f32x2 rd, ra, rb;\n"
      "  mov.b64 {%0, %1}, rd;\n"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

constexpr int FWD2_VSTAGES = 3;  // V is needed one step later than K is released: a third stage hides the load latency
struct Fwd2Bars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[FWD2_VSTAGES], v_empty[FWD2_VSTAGES];
  uint64_t s_full[2], p_ready[2], o_final[2];
  uint32_t tmem_slot;
  int abort_flag;
};

template <int D>
__global__ void __launch_bounds__(384, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  constexpr int KSTEPS = D / 16;
  constexpr uint32_t IDESC_S = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(ATT_BM, D, 0, 1);
  constexpr int TILE_BYTES = 2 * PANEL_BYTES;
  constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
  constexpr int POLY_PAIRS_OF_4 = 0;        // measured: the softmax warps are issue-bound, the polynomial does not pay

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                     // tile A, tile B
  uint8_t* sK = sQ + 2 * TILE_BYTES;      // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;      // FWD2_VSTAGES stages
  Fwd2Bars* bars = reinterpret_cast<Fwd2Bars*>(sV + FWD2_VSTAGES * TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + ATT_BM - 1) / ATT_BM;
  const int npair = (nqb + 1) / 2;
  // grid (heads, pairs, batch): CTAs are issued in linear order, so all heads of the heaviest (latest) pair go first and
  // the lightest pairs fill the tail -- longest-first over the whole grid, not per head
  const int pair = npair - 1 - blockIdx.y;
  const int h = blockIdx.x, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int qbA = 2 * pair, qbB = 2 * pair + 1;
  const int nA = qbA + 1;                       // key blocks of tile A (block qbA is its diagonal)
  const int nB = (qbB < nqb) ? qbB + 1 : 0;     // tile B may not exist (odd number of query blocks)
  const int nmax = max(nA, nB);
  const int xq = h * D, xk = p.wq + hk * D, xv = p.wq + p.wk + hk * D;

  // The TMA thread (warp 8, lane 0) owns the barrier setup so that the Q tiles and the first K block are requested
  // before the CTA-wide sync and the tensor-memory allocation: with one CTA resident per SM nothing else hides the
  // ~2.5 us from launch to the first S.
  if (threadIdx.x == 256) {
    tma_prefetch_desc(&tm);
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < FWD2_VSTAGES; ++i) {
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_ready[i], 4);
      mbar_init(&bars->o_final[i], 1);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    mbar_expect_tx(&bars->q_full, 2 * TILE_BYTES);
    tma_load_3d(sQ, &tm, &bars->q_full, xq, qbA * ATT_BM, b);
    tma_load_3d(sQ + PANEL_BYTES, &tm, &bars->q_full, xq + 64, qbA * ATT_BM, b);
    tma_load_3d(sQ + TILE_BYTES, &tm, &bars->q_full, xq, qbB * ATT_BM, b);   // rows past S read as zero
    tma_load_3d(sQ + TILE_BYTES + PANEL_BYTES, &tm, &bars->q_full, xq + 64, qbB * ATT_BM, b);
    mbar_expect_tx(&bars->k_full[0], TILE_BYTES);
    tma_load_3d(sK, &tm, &bars->k_full[0], xk, 0, b);
    tma_load_3d(sK + PANEL_BYTES, &tm, &bars->k_full[0], xk + 64, 0, b);
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  // warps 0-3: softmax of tile A, 4-7: softmax of tile B, 8: TMA, 9: MMA, 10-11: idle (they complete the third
  // warpgroup so that it can hand its registers to the softmax warpgroups)
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    // lane 0 feeds Q and the K ring, lane 1 the V ring: a stall of one ring does not delay requests of the other
    if (lane == 0) {
      int issued = 1;   // Q and key block 0 went out before the CTA-wide sync
      for (int j = 1; j < nmax; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, &tm, &bars->k_full[s], xk, j * ATT_BN, b);
        tma_load_3d(sK + s * TILE_BYTES + PANEL_BYTES, &tm, &bars->k_full[s], xk + 64, j * ATT_BN, b);
        issued = j + 1;
      }
      // every issued load must land before the CTA exits
      unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->q_full, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      for (int j = max(0, issued - 2); j < issued; ++j) {
        t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->k_full[j & 1], (j >> 1) & 1) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      }
    } else if (lane == 1) {
      int issued = 0;
      for (int j = 0; j < nmax; ++j) {
        const int s = j % FWD2_VSTAGES;
        const uint32_t ph = (j / FWD2_VSTAGES) & 1;
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_3d(sV + s * TILE_BYTES, &tm, &bars->v_full[s], xv, j * ATT_BN, b);
        tma_load_3d(sV + s * TILE_BYTES + PANEL_BYTES, &tm, &bars->v_full[s], xv + 64, j * ATT_BN, b);
        issued = j + 1;
      }
      for (int j = max(0, issued - FWD2_VSTAGES); j < issued; ++j) {
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->v_full[j % FWD2_VSTAGES], (j / FWD2_VSTAGES) & 1) &&
               globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      auto issue_s = [&](int x, int j) {  // S_x = Q_x K_j^T
        const uint32_t kb = aK + (j & 1) * TILE_BYTES, qb = aQ + x * TILE_BYTES;
#pragma unroll
        for (int t = 0; t < KSTEPS; ++t) {
          const uint32_t off = (t >> 2) * PANEL_BYTES + (t & 3) * 32;
          umma_bf16(tmem_base + x * 128, make_smem_desc(qb + off, 16, 1024), make_smem_desc(kb + off, 16, 1024), IDESC_S,
                    t ? 1u : 0u);
        }
        umma_commit(&bars->s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {  // O_x += P_x V_j, P_x in TMEM over the first 64 columns of S_x
        const uint32_t vb = aV + (j % FWD2_VSTAGES) * TILE_BYTES;
#pragma unroll
        for (int t = 0; t < ATT_BN / 16; ++t)
          umma_bf16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + t * 8,
                       make_smem_desc(vb + t * 2048, PANEL_BYTES, 1024), IDESC_O, (j | t) ? 1u : 0u);
      };
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.err, ERR_WAIT_ATTN) &&
                mbar_wait(&bars->k_full[0], 0, abort_flag, p.err, ERR_WAIT_ATTN);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        if (nB > 0) issue_s(1, 0);
        umma_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < nmax && ok; ++j) {
        const int s = j & 1, sv3 = j % FWD2_VSTAGES;
        const uint32_t ph1 = ((j + 1) >> 1) & 1;
        if (!mbar_wait(&bars->v_full[sv3], (j / FWD2_VSTAGES) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
        if (j + 1 < nmax && !mbar_wait(&bars->k_full[s ^ 1], ph1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int nx = x ? nB : nA;
          if (j >= nx) continue;
          if (!mbar_wait(&bars->p_ready[x], j & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
          tc_fence_after();
          issue_pv(x, j);
          if (j + 1 < nx) issue_s(x, j + 1);
          else umma_commit(&bars->o_final[x]);
        }
        if (!ok) break;
        umma_commit(&bars->v_empty[sv3]);
        if (j + 1 < nmax) umma_commit(&bars->k_empty[s ^ 1]);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int x = warp >> 2;                  // 0: tile A, 1: tile B
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qb = x ? qbB : qbA;
    const int nx = x ? nB : nA;
    const int qrow = qb * ATT_BM + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_base + x * 128 + lane_addr;          // S_x (and P_x over its first 64 columns)
    const uint32_t to = tmem_base + 256 + x * 128 + lane_addr;    // O_x
    const float scale_log2 = p.scale_log2;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nx && ok; ++j) {
      if (!mbar_wait(&bars->s_full[x], j & 1, abort_flag, p.err, ERR_WAIT_ATTN)) { ok = false; break; }
      tc_fence_after();
      float sv[ATT_BN];
#pragma unroll
      for (int c = 0; c < ATT_BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(ts + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[c + i] = __uint_as_float(v[i]);
      }
      tmem_ld_wait();
      if (j == qb) {  // diagonal block: keys beyond the query (this also covers keys past the end of the sequence)
        const int limit = qrow - j * ATT_BN;
#pragma unroll
        for (int i = 0; i < ATT_BN; ++i)
          if (i > limit) sv[i] = -INFINITY;
      }
      float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};  // four independent chains of three-input max
#pragma unroll
      for (int i = 4; i + 7 < ATT_BN; i += 8) {
        mx4[0] = fmax3(mx4[0], sv[i], sv[i + 1]);
        mx4[1] = fmax3(mx4[1], sv[i + 2], sv[i + 3]);
        mx4[2] = fmax3(mx4[2], sv[i + 4], sv[i + 5]);
        mx4[3] = fmax3(mx4[3], sv[i + 6], sv[i + 7]);
      }
      mx4[0] = fmax3(mx4[0], sv[ATT_BN - 4], sv[ATT_BN - 3]);
      mx4[1] = fmax3(mx4[1], sv[ATT_BN - 2], sv[ATT_BN - 1]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * scale_log2);
      // raise the reference max only when it moved by more than the threshold (decided per warp: the TMEM accesses of
      // the rescale are warp-collective)
      const bool grow = (m_new - m > RESCALE_THRESHOLD) || (m == -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - m_new);
        if (j > 0) {
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(to + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(to + c, v);
          }
        }
        l *= alpha;
        m = m_new;
      }
      const float2 neg_m2 = make_float2(-m, -m), scale2 = make_float2(scale_log2, scale_log2);
      float2 rs[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c = 0; c < ATT_BN; c += 32) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 a = ffma2(make_float2(sv[c + i], sv[c + i + 1]), scale2, neg_m2);
          // POLY_PAIRS_OF_4 pairs in four go through the polynomial (FMA pipe) instead of the MUFU
          const bool poly = POLY_PAIRS_OF_4 > 0 && ((i >> 1) & 3) < POLY_PAIRS_OF_4;
          const float2 pr = make_float2(poly ? ex2_poly(a.x) : ex2_approx(a.x), poly ? ex2_poly(a.y) : ex2_approx(a.y));
          rs[(i >> 1) & 3] = fadd2(rs[(i >> 1) & 3], pr);
          packed[i >> 1] = pack_bf16x2(pr.x, pr.y);
        }
        tmem_st_32x16(ts + (c >> 1), packed);
      }
      {
        const float2 t = fadd2(fadd2(rs[0], rs[1]), fadd2(rs[2], rs[3]));
        l += t.x + t.y;
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[x]);
    }
    if (ok && nx > 0) {
      if (mbar_wait(&bars->o_final[x], 0, abort_flag, p.err, ERR_WAIT_ATTN)) {
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.o + (static_cast<size_t>(b) * p.S + qrow) * (p.H * D) + h * D;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(to + c, v);
          tmem_ld_wait();
          if (qrow < p.S) {
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              o[i >> 1] = pack_bf16x2(__uint_as_float(v[i]) * inv_l, __uint_as_float(v[i + 1]) * inv_l);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(orow + c + 8 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
          }
        }
        if (qrow < p.S && p.lse)
          p.lse[(static_cast<size_t>(b) * p.H + h) * p.S + qrow] = (m + log2f(l)) * 0.6931471805599453f;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ backward
struct BwdBars {
  uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_ready, dq_full, dq_empty;
  uint32_t tmem_slot;
  int abort_flag;
};

struct AttnBwdParams {
  int B, S, H, Hkv, D, wq, wk;
  float scale, scale_log2;
  const float* lse;     // [B, H, S]
  const float* delta;   // [B, H, S]  rowsum(dO * O)
  float* dq_acc;        // [B, S, H*D] fp32, zero on entry; receives sum over key blocks of dS K (unscaled)
  __nv_bfloat16* dqkv;  // packed [B, S, (H + 2 Hkv) * D]; this kernel writes the k and v sections
  int* err;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// write 32 consecutive bf16 of row r (columns c .. c+31 of a [128 x 128] tile) into a K-major 128B-swizzled tile
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int r, int c, const uint32_t (&packed)[16]) {
  uint8_t* prow = tile + (c >> 6) * PANEL_BYTES + r * 128;
  const int chunk0 = (c & 63) >> 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int phys = (chunk0 + q) ^ (r & 7);
    *reinterpret_cast<uint4*>(prow + phys * 16) =
        make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
  }
}

template <int D>
__global__ void __launch_bounds__(192, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
  constexpr int KSTEPS_D = D / 16;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, 0, 0);   // S = Q K^T, dP = dO V^T
  constexpr uint32_t IDESC_TT = make_idesc_bf16(128, D, 1, 1);     // dV += P^T dO, dK += dS^T Q
  constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, D, 0, 1);     // dQ = dS K
  constexpr int TILE_BYTES = 2 * PANEL_BYTES;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sP = sdO + TILE_BYTES;
  uint8_t* sdS = sP + TILE_BYTES;
  BwdBars* bars = reinterpret_cast<BwdBars*>(sdS + TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int rep = p.H / p.Hkv;
  const int nqb = (p.S + ATT_BM - 1) / ATT_BM;
  const int per_head = nqb - kvb;            // query blocks at or below the diagonal
  const int n_it = rep * per_head;
  const int k0 = kvb * ATT_BN;
  const int xk = p.wq + hk * D, xv = p.wq + p.wk + hk * D;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    mbar_init(&bars->qdo_full, 1);
    mbar_init(&bars->qdo_empty, 1);
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->pds_ready, 4);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_empty, 4);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQKV);
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
      tma_load_3d(sK, &tmQKV, &bars->kv_full, xk, k0, b);
      tma_load_3d(sK + PANEL_BYTES, &tmQKV, &bars->kv_full, xk + 64, k0, b);
      tma_load_3d(sV, &tmQKV, &bars->kv_full, xv, k0, b);
      tma_load_3d(sV + PANEL_BYTES, &tmQKV, &bars->kv_full, xv + 64, k0, b);
      int issued = 0;
      for (int it = 0; it < n_it; ++it) {
        const int h = hk * rep + it / per_head;
        const int q0 = (kvb + it % per_head) * ATT_BM;
        if (!mbar_wait(&bars->qdo_empty, (it & 1) ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        mbar_expect_tx(&bars->qdo_full, 2 * TILE_BYTES);
        tma_load_3d(sQ, &tmQKV, &bars->qdo_full, h * D, q0, b);
        tma_load_3d(sQ + PANEL_BYTES, &tmQKV, &bars->qdo_full, h * D + 64, q0, b);
        tma_load_3d(sdO, &tmDO, &bars->qdo_full, h * D, q0, b);
        tma_load_3d(sdO + PANEL_BYTES, &tmDO, &bars->qdo_full, h * D + 64, q0, b);
        issued = it + 1;
      }
      unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->kv_full, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      if (issued > 0) {
        t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->qdo_full, (issued - 1) & 1) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sdO), aP = smem_u32(sP),
                     aDS = smem_u32(sdS);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(&bars->qdo_full, ph, abort_flag, p.err, ERR_WAIT_ATTN) ||
            !mbar_wait(&bars->dq_empty, ph ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < KSTEPS_D; ++t) {
          const uint32_t off = (t >> 2) * PANEL_BYTES + (t & 3) * 32;
          umma_bf16(tmem_base + COL_S, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024),
                    IDESC_QK, t ? 1u : 0u);
        }
#pragma unroll
        for (int t = 0; t < KSTEPS_D; ++t) {
          const uint32_t off = (t >> 2) * PANEL_BYTES + (t & 3) * 32;
          umma_bf16(tmem_base + COL_DP, make_smem_desc(aDO + off, 16, 1024), make_smem_desc(aV + off, 16, 1024),
                    IDESC_QK, t ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full);
        if (!mbar_wait(&bars->pds_ready, ph, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 8; ++t) {  // contraction over the 128 query rows, 16 per step
          const uint64_t aPt = make_smem_desc(aP + t * 2048, PANEL_BYTES, 1024);     // P^T  (MN-major A)
          const uint64_t aSt = make_smem_desc(aDS + t * 2048, PANEL_BYTES, 1024);    // dS^T (MN-major A)
          const uint64_t bDO = make_smem_desc(aDO + t * 2048, PANEL_BYTES, 1024);    // dO   (MN-major B)
          const uint64_t bQ = make_smem_desc(aQ + t * 2048, PANEL_BYTES, 1024);      // Q    (MN-major B)
          umma_bf16(tmem_base + COL_DV, aPt, bDO, IDESC_TT, (it | t) ? 1u : 0u);
          umma_bf16(tmem_base + COL_DK, aSt, bQ, IDESC_TT, (it | t) ? 1u : 0u);
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) {  // contraction over the 128 keys
          const uint64_t aS = make_smem_desc(aDS + (t >> 2) * PANEL_BYTES + (t & 3) * 32, 16, 1024);
          const uint64_t bK = make_smem_desc(aK + t * 2048, PANEL_BYTES, 1024);      // K (MN-major B)
          umma_bf16(tmem_base + COL_S, aS, bK, IDESC_DQ, t ? 1u : 0u);
        }
        umma_commit(&bars->dq_full);
        umma_commit(&bars->qdo_empty);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool elected = (warp == 2 && lane == 0);   // issues the bulk reductions of dQ
    uint8_t* stage = sP;                             // dQ staging (fp32, D/32 boxes of 16 KB) over the P and dS tiles
    bool ok = true;
    // The four warps meet at named barrier 1 twice per iteration; nobody leaves the loop between two meetings on a
    // private decision: a failed wait raises the CTA abort flag, which everyone reads right after the barrier.
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = it & 1;
      const int h = hk * rep + it / per_head;
      const int qb = kvb + it % per_head;
      const int qrow = qb * ATT_BM + r;
      const bool row_ok = qrow < p.S;
      const size_t stat = (static_cast<size_t>(b) * p.H + h) * p.S + qrow;
      const float lse2 = row_ok ? p.lse[stat] * 1.4426950408889634f : 0.f;
      const float delta = row_ok ? p.delta[stat] : 0.f;
      ok = mbar_wait(&bars->sdp_full, ph, abort_flag, p.err, ERR_WAIT_ATTN);
      if (elected) bulk_wait_read_all();             // the previous dQ tile has left the staging area
      named_barrier_sync(1, 128);
      if (*abort_flag) { ok = false; break; }
      tc_fence_after();
      const bool diag = (qb == kvb);
#pragma unroll 1
      for (int c = 0; c < ATT_BN; c += 32) {
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32(tmem_base + COL_S + lane_addr + c, sv);
        tmem_ld_32x32(tmem_base + COL_DP + lane_addr + c, dpv);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = 0.f, p1 = 0.f;
          if (row_ok) {
            if (!(diag && (k0 + c + i > qrow))) p0 = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - lse2);
            if (!(diag && (k0 + c + i + 1 > qrow))) p1 = exp2f(__uint_as_float(sv[i + 1]) * p.scale_log2 - lse2);
          }
          pp[i >> 1] = pack_bf16x2(p0, p1);
          ds[i >> 1] = pack_bf16x2(p0 * (__uint_as_float(dpv[i]) - delta), p1 * (__uint_as_float(dpv[i + 1]) - delta));
        }
        store_row_chunk_sw128(sP, r, c, pp);
        store_row_chunk_sw128(sdS, r, c, ds);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready);
      ok = mbar_wait(&bars->dq_full, ph, abort_flag, p.err, ERR_WAIT_ATTN);
      if (ok) {
        // dQ tile: TMEM -> fp32 staging in shared memory (128-byte swizzle, boxes of 32 columns), then ONE bulk
        // tensor reduction per box adds it to the global accumulator (rows past the sequence end are clipped)
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + COL_S + lane_addr + c, v);
          tmem_ld_wait();
          uint8_t* row = stage + (c >> 5) * PANEL_BYTES + r * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(row + ((q ^ (r & 7)) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        tc_fence_before();
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->dq_empty);
      named_barrier_sync(1, 128);
      if (*abort_flag) { ok = false; break; }
      if (elected) {
#pragma unroll
        for (int c = 0; c < D; c += 32)
          tma_reduce_add_3d(&tmDQ, stage + (c >> 5) * PANEL_BYTES, h * D + c, qb * ATT_BM, b);
        bulk_commit_group();
      }
    }
    if (elected) bulk_wait_all();
    if (ok && n_it > 0) {
      // all MMAs are complete (the last dq_full was waited on): write dV and scale * dK for this key block
      const int key = k0 + r;
      const size_t wtot = static_cast<size_t>(p.wq) + 2 * p.wk;
      __nv_bfloat16* dk_row = p.dqkv + (static_cast<size_t>(b) * p.S + key) * wtot + p.wq + hk * D;
      __nv_bfloat16* dv_row = dk_row + p.wk;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t v[16], k[16];
        tmem_ld_32x16(tmem_base + COL_DV + lane_addr + c, v);
        tmem_ld_32x16(tmem_base + COL_DK + lane_addr + c, k);
        tmem_ld_wait();
        if (key < p.S) {
          uint32_t ov[8], ok2[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            ov[i >> 1] = pack_bf16x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            ok2[i >> 1] = pack_bf16x2(__uint_as_float(k[i]) * p.scale, __uint_as_float(k[i + 1]) * p.scale);
          }
          *reinterpret_cast<uint4*>(dv_row + c) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
          *reinterpret_cast<uint4*>(dv_row + c + 8) = make_uint4(ov[4], ov[5], ov[6], ov[7]);
          *reinterpret_cast<uint4*>(dk_row + c) = make_uint4(ok2[0], ok2[1], ok2[2], ok2[3]);
          *reinterpret_cast<uint4*>(dk_row + c + 8) = make_uint4(ok2[4], ok2[5], ok2[6], ok2[7]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ backward, v2
// Transposed formulation: one CTA per (128-key block, kv head, batch) computes, for every query block i at or below
// the diagonal (and every query head of the group),
//     S^T  = K Q_i^T      dP^T = V dO_i^T          [key lanes x query columns] in TMEM
//     P^T  = exp2(S^T scale - lse_q)               bf16, written over the consumed S^T columns (TMEM)
//     dS^T = P^T (dP^T - delta_q)                  bf16, written over the consumed dP^T columns (TMEM) and to smem
//     dV  += P^T dO_i     dK += dS^T Q_i           A operand straight from TMEM, accumulators in TMEM for the whole loop
//     dQ_i = dS K                                  A = dS^T tile in smem read MN-major; added to the fp32 accumulator
// so P never touches shared memory, the softmax needs no row reductions (lse and delta are per column), and the 32 KB
// saved hold a second stage of Q_i / dO_i tiles: the next block's loads overlap this block's work.
// Warps: 0 TMA, 1 / 10 / 11 MMA issuers, 2-9 softmax (two threads per key row, 64 query columns each).
// TMEM: ST [0,128): P^T packs into [0,32) and [96,128), dQ columns 0..63 go to the hole [32,96);
//       DPT [128,256): dS^T packs into [128,160) and [224,256), dQ columns 64..D-1 go to [160,224);
//       dV [256,256+D), dK [384,384+D).
constexpr int BWD2_SLOTS = 4;   // Q_i, dO_i, Q_i+1, dO_i+1
struct Bwd2Bars {
  uint64_t kv_full, slot_full[BWD2_SLOTS], slot_empty[BWD2_SLOTS], sdp_full, pds_ready, dq_full, dq_empty;
  uint32_t tmem_slot;
  int abort_flag;
};

template <int D>
__global__ void __launch_bounds__(384, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                 const AttnBwdParams p) {
  constexpr int KSTEPS_D = D / 16;
  constexpr uint32_t IDESC_ST = make_idesc_bf16(128, 128, 0, 0);     // S^T = K Q^T, dP^T = V dO^T
  constexpr uint32_t IDESC_ACC = make_idesc_bf16(128, D, 0, 1);      // dV += P^T dO, dK += dS^T Q  (A in TMEM)
  constexpr uint32_t IDESC_DQA = make_idesc_bf16(128, 64, 1, 1);     // dQ[:, 0:64) = dS K
  constexpr int DQB = D - 64;                                        // second piece of dQ (0, 32 or 64 columns)
  constexpr uint32_t IDESC_DQB = make_idesc_bf16(128, DQB > 0 ? DQB : 16, 1, 1);
  constexpr int TILE_BYTES = 2 * PANEL_BYTES;
  constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;
  constexpr uint32_t COL_DQA = 32, COL_DQB = 160;

  // 7 tiles of 32 KB leave no room for alignment slack: the dynamic shared window itself must be 1024-byte aligned
  // (it is when the kernel has no static shared memory); a CTA that finds it otherwise reports and leaves.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, ERR_WAIT_ATTN);
    return;
  }
  uint8_t* smem = smem_raw;
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sdS = sV + TILE_BYTES;
  uint8_t* sSlot = sdS + TILE_BYTES;                       // BWD2_SLOTS tiles
  float* s_stat = reinterpret_cast<float*>(sSlot + BWD2_SLOTS * TILE_BYTES);   // [2 parities][lse2 | delta][128]
  Bwd2Bars* bars = reinterpret_cast<Bwd2Bars*>(s_stat + 2 * 2 * 128);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (kv heads, key blocks, batch): key block 0 meets every query block, the last one a single block; in linear
  // order all heads of the heaviest key block go first (longest-first over the whole grid)
  const int kvb = blockIdx.y, hk = blockIdx.x, b = blockIdx.z;
  const int rep = p.H / p.Hkv;
  const int nqb = (p.S + ATT_BM - 1) / ATT_BM;
  const int per_head = nqb - kvb;
  const int n_it = rep * per_head;
  const int k0 = kvb * ATT_BN;
  const int xk = p.wq + hk * D, xv = p.wq + p.wk + hk * D;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int i = 0; i < BWD2_SLOTS; ++i) {
      mbar_init(&bars->slot_full[i], 1);
      mbar_init(&bars->slot_empty[i], 1);
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->pds_ready, 8);
    mbar_init(&bars->dq_full, 2);   // the dV/dK issuer and the dQ issuer each commit once
    mbar_init(&bars->dq_empty, 8);
    bars->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    // this thread is also the TMA thread: the K / V tiles are requested before the CTA-wide sync and the TMEM allocation
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
    mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
    tma_load_3d(sK, &tmQKV, &bars->kv_full, xk, k0, b);
    tma_load_3d(sK + PANEL_BYTES, &tmQKV, &bars->kv_full, xk + 64, k0, b);
    tma_load_3d(sV, &tmQKV, &bars->kv_full, xv, k0, b);
    tma_load_3d(sV + PANEL_BYTES, &tmQKV, &bars->kv_full, xv + 64, k0, b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;   // tiles (two per iteration: Q then dO)
      for (int t = 0; t < 2 * n_it; ++t) {
        const int it = t >> 1;
        const int h = hk * rep + it / per_head;
        const int q0 = (kvb + it % per_head) * ATT_BM;
        const int slot = t % BWD2_SLOTS;
        if (!mbar_wait(&bars->slot_empty[slot], ((t / BWD2_SLOTS) & 1) ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
        uint8_t* dst = sSlot + slot * TILE_BYTES;
        mbar_expect_tx(&bars->slot_full[slot], TILE_BYTES);
        if (t & 1) {
          tma_load_3d(dst, &tmDO, &bars->slot_full[slot], h * D, q0, b);
          tma_load_3d(dst + PANEL_BYTES, &tmDO, &bars->slot_full[slot], h * D + 64, q0, b);
        } else {
          tma_load_3d(dst, &tmQKV, &bars->slot_full[slot], h * D, q0, b);
          tma_load_3d(dst + PANEL_BYTES, &tmQKV, &bars->slot_full[slot], h * D + 64, q0, b);
        }
        issued = t + 1;
      }
      unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->kv_full, 0) && globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      for (int t = max(0, issued - BWD2_SLOTS); t < issued; ++t) {
        t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->slot_full[t % BWD2_SLOTS], (t / BWD2_SLOTS) & 1) &&
               globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
      }
    }
  } else if (warp == 1 || warp >= 10) {
    // Three MMA issuers, one per dependency chain: warp 1 issues S^T and dP^T (needs only Q / dO in shared memory),
    // warp 10 dV and dK (needs P^T / dS^T in tensor memory), warp 11 dQ (needs dS^T in shared memory).  A single issuer
    // blocks on one chain's barrier while another chain's MMAs could already run: S^T / dP^T of the next query block
    // now start while the softmax warps still hold this block's dQ (measured 1.13 -> 1.04 ms on the flagship shape).
    if (lane == 0) {
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDS = smem_u32(sdS), aSlot = smem_u32(sSlot);
      const uint64_t dKk = make_smem_desc(aK, 16, 1024), dVk = make_smem_desc(aV, 16, 1024);          // K-major A
      const uint64_t dKm = make_smem_desc(aK, PANEL_BYTES, 1024);                                     // MN-major B
      const uint64_t dSm = make_smem_desc(aDS, PANEL_BYTES, 1024);                                    // MN-major A
      bool ok = (warp != 1) || mbar_wait(&bars->kv_full, 0, abort_flag, p.err, ERR_WAIT_ATTN);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ph = it & 1;
        const int tq = 2 * it, tdo = 2 * it + 1;
        const uint32_t aQ = aSlot + (tq % BWD2_SLOTS) * TILE_BYTES, aDO = aSlot + (tdo % BWD2_SLOTS) * TILE_BYTES;
        if (warp == 1) {
          if (!mbar_wait(&bars->slot_full[tq % BWD2_SLOTS], (tq / BWD2_SLOTS) & 1, abort_flag, p.err, ERR_WAIT_ATTN) ||
              !mbar_wait(&bars->dq_empty, ph ^ 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after();
          const uint64_t dQk = make_smem_desc(aQ, 16, 1024);
#pragma unroll
          for (int t = 0; t < KSTEPS_D; ++t) {
            const uint32_t off = ((t >> 2) * PANEL_BYTES + (t & 3) * 32) >> 4;
            umma_bf16(tmem_base + COL_ST, dKk + off, dQk + off, IDESC_ST, t ? 1u : 0u);
          }
          if (!mbar_wait(&bars->slot_full[tdo % BWD2_SLOTS], (tdo / BWD2_SLOTS) & 1, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after();
          const uint64_t dDOk = make_smem_desc(aDO, 16, 1024);
#pragma unroll
          for (int t = 0; t < KSTEPS_D; ++t) {
            const uint32_t off = ((t >> 2) * PANEL_BYTES + (t & 3) * 32) >> 4;
            umma_bf16(tmem_base + COL_DPT, dVk + off, dDOk + off, IDESC_ST, t ? 1u : 0u);
          }
          umma_commit(&bars->sdp_full);
        } else if (warp == 10) {
          if (!mbar_wait(&bars->pds_ready, ph, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after();
          const uint64_t dDOm = make_smem_desc(aDO, PANEL_BYTES, 1024), dQm = make_smem_desc(aQ, PANEL_BYTES, 1024);
#pragma unroll
          for (int t = 0; t < 8; ++t) {  // contraction over the 128 queries, 16 per step = 8 packed TMEM columns
            const uint32_t pcol = (t < 4) ? t * 8 : 96 + (t - 4) * 8;
            umma_bf16_ts(tmem_base + COL_DV, tmem_base + COL_ST + pcol, dDOm + t * (2048 >> 4), IDESC_ACC, (it | t) ? 1u : 0u);
            umma_bf16_ts(tmem_base + COL_DK, tmem_base + COL_DPT + pcol, dQm + t * (2048 >> 4), IDESC_ACC, (it | t) ? 1u : 0u);
          }
          umma_commit(&bars->dq_full);
          umma_commit(&bars->slot_empty[tq % BWD2_SLOTS]);
          umma_commit(&bars->slot_empty[tdo % BWD2_SLOTS]);
        } else if (warp == 11) {
          if (!mbar_wait(&bars->pds_ready, ph, abort_flag, p.err, ERR_WAIT_ATTN)) break;
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 8; ++t) {  // contraction over the 128 keys; A = dS^T tile read MN-major (M = queries)
            umma_bf16(tmem_base + COL_DQA, dSm + t * (2048 >> 4), dKm + t * (2048 >> 4), IDESC_DQA, t ? 1u : 0u);
            if constexpr (DQB > 0)
              umma_bf16(tmem_base + COL_DQB, dSm + t * (2048 >> 4), dKm + ((PANEL_BYTES + t * 2048) >> 4), IDESC_DQB,
                        t ? 1u : 0u);
          }
          umma_commit(&bars->dq_full);
        }
      }
    }
  } else {
    // warps 2..9: TMEM lane quadrant = warp % 4; the two warps with the same quadrant split the query columns
    const int quad = warp & 3;
    const int hsel = (warp - 2) >> 2;         // 0: warps 2-5 (query columns 0..63), 1: warps 6-9 (64..127)
    const int r = quad * 32 + lane;           // key row (phase A) / query row (phase B)
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int wt = threadIdx.x - 64;          // 0..255 inside the softmax group
    const int key = k0 + r;
    // statistics of the first query block
    auto load_stat = [&](int it) -> float {
      const int h = hk * rep + it / per_head;
      const int q = (kvb + it % per_head) * ATT_BM + (wt & 127);
      if (it >= n_it || q >= p.S) return 0.f;
      const size_t idx = (static_cast<size_t>(b) * p.H + h) * p.S + q;
      return (wt < 128) ? p.lse[idx] * 1.4426950408889634f : p.delta[idx];
    };
    float stat_next = load_stat(0);
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = it & 1;
      const int h = hk * rep + it / per_head;
      const int qb = kvb + it % per_head;
      const int q0 = qb * ATT_BM;
      float* st = s_stat + ph * 256;
      st[wt] = stat_next;                      // [0,128): lse * log2(e), [128,256): delta of this query block
      stat_next = load_stat(it + 1);           // prefetch for the next block
      mbar_wait(&bars->sdp_full, ph, abort_flag, p.err, ERR_WAIT_ATTN);
      named_barrier_sync(1, 256);              // statistics visible; uniform abort decision
      if (*abort_flag) break;
      tc_fence_after();
      const bool diag = (qb == kvb);
      const int nvalid = p.S - q0;             // query columns at or past nvalid do not exist
      // this thread's 64 query columns, in two chunks of 32; the upper half walks downwards so that its packed
      // stores (into the top of its own column range) never land on columns it has not read yet
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = hsel ? (96 - 32 * cc) : 32 * cc;
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32(tmem_base + COL_ST + lane_addr + c, sv);
        tmem_ld_32x32(tmem_base + COL_DPT + lane_addr + c, dpv);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 l2 = *reinterpret_cast<const float2*>(st + c + i);
          const float2 dl = *reinterpret_cast<const float2*>(st + 128 + c + i);
          float p0 = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -l2.x));
          float p1 = ex2_approx(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -l2.y));
          if ((diag && key > q0 + c + i) || c + i >= nvalid) p0 = 0.f;
          if ((diag && key > q0 + c + i + 1) || c + i + 1 >= nvalid) p1 = 0.f;
          pp[i >> 1] = pack_bf16x2(p0, p1);
          ds[i >> 1] = pack_bf16x2(p0 * (__uint_as_float(dpv[i]) - dl.x), p1 * (__uint_as_float(dpv[i + 1]) - dl.y));
        }
        const uint32_t pcol = (hsel ? 96 + ((c - 64) >> 1) : (c >> 1));
        tmem_st_32x16(tmem_base + COL_ST + lane_addr + pcol, pp);
        tmem_st_32x16(tmem_base + COL_DPT + lane_addr + pcol, ds);
        store_row_chunk_sw128(sdS, r, c, ds);  // dS^T tile [key rows][query columns] for the dQ MMA
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready);
      mbar_wait(&bars->dq_full, ph, abort_flag, p.err, ERR_WAIT_ATTN);
      if (!*abort_flag) {
        // dQ tile [query lanes x D]: warps 2-5 take columns 0..63, warps 6-9 columns 64..D-1
        tc_fence_after();
        // accumulator layout [b, h, query block, D/4, 128 rows, 4]: for one group of 4 columns the 128 rows are
        // contiguous, so the 32 lanes of a reduction instruction cover 512 contiguous bytes
        const int qrow = q0 + r;
        float* dq_blk = p.dq_acc + ((static_cast<size_t>(b) * p.H + h) * nqb + qb) * (static_cast<size_t>(D) * ATT_BM) + r * 4;
        const int ncols = hsel ? DQB : 64;
        const uint32_t src = tmem_base + (hsel ? COL_DQB : COL_DQA) + lane_addr;
        const int dcol0 = hsel ? 64 : 0;
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
          if (c < ncols) {
            uint32_t v[16];
            tmem_ld_32x16(src + c, v);
            tmem_ld_wait();
            if (qrow < p.S) {
#pragma unroll
              for (int i = 0; i < 16; i += 4)
                red_add_v4(dq_blk + ((dcol0 + c + i) >> 2) * (ATT_BM * 4), __uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                           __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            }
          }
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->dq_empty);
    }
    if (!*abort_flag && n_it > 0) {
      // the last dq_full wait covered every MMA: write dV and scale * dK of this key block
      const size_t wtot = static_cast<size_t>(p.wq) + 2 * p.wk;
      __nv_bfloat16* base_row = p.dqkv + (static_cast<size_t>(b) * p.S + key) * wtot + p.wq + hk * D;
      // warps 2-5 write dV, warps 6-9 write scale * dK
      const uint32_t src = tmem_base + (hsel ? COL_DK : COL_DV) + lane_addr;
      __nv_bfloat16* dst = base_row + (hsel ? 0 : p.wk);
      const float mul = hsel ? p.scale : 1.f;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t v[16];
        tmem_ld_32x16(src + c, v);
        tmem_ld_wait();
        if (key < p.S) {
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2)
            o[i >> 1] = pack_bf16x2(__uint_as_float(v[i]) * mul, __uint_as_float(v[i + 1]) * mul);
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H, int D) {
  const size_t w = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<size_t>(B) * S * H) return;
  const int h = static_cast<int>(w % H);
  const size_t bs = w / H;
  const __nv_bfloat16* op = o + (bs * H + h) * D;
  const __nv_bfloat16* dp = d_o + (bs * H + h) * D;
  float acc = 0.f;
  for (int i = lane; i < D; i += 32) acc += bf2f(op[i]) * bf2f(dp[i]);
  acc = warp_sum(acc);
  if (lane == 0) delta[(static_cast<size_t>(bs / S) * H + h) * S + bs % S] = acc;
}

// Same for the block-interleaved accumulator of the v2 backward ([b, h, query block, D/4, 128 rows, 4]): one CTA per
// (query block, head, batch) reads its D x 128 floats coalesced, transposes through shared memory, writes bf16 rows.
template <int D>
__global__ void __launch_bounds__(256)
attn_dq_convert_blocked_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int S, int H, int wtot,
                               float scale) {
  constexpr int ROWS = 64;   // half a query block per CTA (static shared memory limit)
  __shared__ float tile[ROWS][D + 1];
  const int qb = blockIdx.x >> 1, r0 = (blockIdx.x & 1) * ROWS, h = blockIdx.y, b = blockIdx.z;
  const int nqb = gridDim.x >> 1;
  const float4* src = reinterpret_cast<const float4*>(
      dq_acc + ((static_cast<size_t>(b) * H + h) * nqb + qb) * (static_cast<size_t>(D) * ATT_BM));
  for (int i = threadIdx.x; i < (D / 4) * ROWS; i += blockDim.x) {
    const int g = i / ROWS, r = i % ROWS;
    const float4 v = src[g * ATT_BM + r0 + r];
    tile[r][4 * g] = v.x; tile[r][4 * g + 1] = v.y; tile[r][4 * g + 2] = v.z; tile[r][4 * g + 3] = v.w;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * (D / 2); i += blockDim.x) {
    const int r = i / (D / 2), c = (i % (D / 2)) * 2;
    const int q = qb * ATT_BM + r0 + r;
    if (q < S)
      *reinterpret_cast<uint32_t*>(dqkv + (static_cast<size_t>(b) * S + q) * wtot + h * D + c) =
          pack_bf16x2(tile[r][c] * scale, tile[r][c + 1] * scale);
  }
}

// dqkv[:, :, 0:wq] = bf16(scale * dq_acc)
__global__ void attn_dq_convert_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, size_t rows,
                                       int wq, int wtot, float scale) {
  const int vpr = wq >> 2;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= rows * vpr) return;
  const size_t row = gid / vpr;
  const int c = static_cast<int>(gid % vpr) << 2;
  const float4 v = *reinterpret_cast<const float4*>(dq_acc + row * wq + c);
  *reinterpret_cast<uint2*>(dqkv + row * wtot + c) =
      make_uint2(pack_bf16x2(v.x * scale, v.y * scale), pack_bf16x2(v.z * scale, v.w * scale));
}

}  // namespace b200


using namespace b200;

template <int D>
static int launch_attn_fwd(const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  constexpr int SMEM = 6 * 2 * PANEL_BYTES + 1024 + 1024;  // Q + 2 K + 2 V + P tiles, barriers, alignment slack
  auto kern = attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  dim3 grid((p.S + ATT_BM - 1) / ATT_BM, p.H, p.B);
  kern<<<grid, 192, SMEM, st>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <int D>
static int launch_attn_fwd2(const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  constexpr int SMEM = (4 + FWD2_VSTAGES) * 2 * PANEL_BYTES + 1024 + 512;  // Q_A, Q_B, 2 x K, 3 x V, barriers
  auto kern = attn_fwd2_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  const int nqb = (p.S + ATT_BM - 1) / ATT_BM;
  dim3 grid(p.H, (nqb + 1) / 2, p.B);
  kern<<<grid, 384, SMEM, st>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int g_attn_fwd_variant = 2;
// 1: one query tile per CTA, P through shared memory; 2: two query tiles per CTA, P in tensor memory (default).
B200_API int b200_attn_set_fwd_variant(int v) {
  const int old = g_attn_fwd_variant;
  if (v == 1 || v == 2) g_attn_fwd_variant = v;
  return old;
}

// qkv: packed rotated [B, S, (H + 2 Hkv) * D] bf16; o: [B, S, H*D] bf16; lse: [B, H, S] fp32 (natural log).
B200_API int b200_attn_fwd(const void* qkv, void* o, float* lse, int B, int S, int H, int Hkv, int D, float scale,
                           void* stream, int* err) {
  if (D % 16 || D > 128 || D < 16 || H % Hkv) return -1;
  const int wtot = (H + 2 * Hkv) * D;
  CUtensorMap tm;
  int rc = make_tmap_3d_bf16(&tm, qkv, wtot, S, B, static_cast<uint64_t>(wtot) * 2, static_cast<uint64_t>(S) * wtot * 2,
                             64, 128);
  if (rc) return rc;
  AttnParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.D = D; p.wq = H * D; p.wk = Hkv * D;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = reinterpret_cast<__nv_bfloat16*>(o); p.lse = lse; p.err = err;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (g_attn_fwd_variant == 2) {
    switch (D) {
      case 64: return launch_attn_fwd2<64>(tm, p, st);
      case 96: return launch_attn_fwd2<96>(tm, p, st);
      case 128: return launch_attn_fwd2<128>(tm, p, st);
      default: return -1;
    }
  }
  switch (D) {
    case 64: return launch_attn_fwd<64>(tm, p, st);
    case 96: return launch_attn_fwd<96>(tm, p, st);
    case 128: return launch_attn_fwd<128>(tm, p, st);
    default: return -1;
  }
}


template <int D>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdParams& p,
                           cudaStream_t st) {
  constexpr int SMEM = 6 * 2 * PANEL_BYTES + 1024 + 1024;  // K, V, Q, dO, P, dS tiles
  auto kern = attn_bwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  dim3 grid((p.S + ATT_BN - 1) / ATT_BN, p.Hkv, p.B);
  kern<<<grid, 192, SMEM, st>>>(tq, tdo, tdq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <int D>
static int launch_attn_bwd2(const CUtensorMap& tq, const CUtensorMap& tdo, const AttnBwdParams& p, cudaStream_t st) {
  constexpr int SMEM = (3 + BWD2_SLOTS) * 2 * PANEL_BYTES + 2048 + 256;  // K, V, dS^T, 4 Q/dO slots, statistics, barriers
  auto kern = attn_bwd2_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  dim3 grid(p.Hkv, (p.S + ATT_BN - 1) / ATT_BN, p.B);
  kern<<<grid, 384, SMEM, st>>>(tq, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int g_attn_bwd_variant = 2;
// 1: query-major tiles, P and dS through shared memory, dQ by bulk tensor reductions;
// 2: transposed tiles, P^T / dS^T in tensor memory, double-buffered Q / dO (default).
B200_API int b200_attn_set_bwd_variant(int v) {
  const int old = g_attn_bwd_variant;
  if (v == 1 || v == 2) g_attn_bwd_variant = v;
  return old;
}

// Backward of b200_attn_fwd.  qkv, o, d_o as in the forward; lse from the forward; delta: scratch [B, H, S] fp32;
// dq_acc: scratch of B * H * ceil(S/128) * 128 * D floats that must be ZERO on entry; dqkv: output, packed like qkv.
B200_API int b200_attn_bwd(const void* qkv, const void* o, const void* d_o, const float* lse, float* delta,
                           float* dq_acc, void* dqkv, int B, int S, int H, int Hkv, int D, float scale, void* stream,
                           int* err) {
  if (D % 16 || D > 128 || D < 16 || H % Hkv) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int wtot = (H + 2 * Hkv) * D, wq = H * D;
  CUtensorMap tq, tdo;
  int rc = make_tmap_3d_bf16(&tq, qkv, wtot, S, B, static_cast<uint64_t>(wtot) * 2, static_cast<uint64_t>(S) * wtot * 2,
                             64, 128);
  if (rc) return rc;
  rc = make_tmap_3d_bf16(&tdo, d_o, wq, S, B, static_cast<uint64_t>(wq) * 2, static_cast<uint64_t>(S) * wq * 2, 64, 128);
  if (rc) return rc;
  CUtensorMap tdq;  // fp32 accumulator [B, S, H*D], boxes of 32 columns x 128 rows
  rc = make_tmap_3d(&tdq, dq_acc, wq, S, B, static_cast<uint64_t>(wq) * 4, static_cast<uint64_t>(S) * wq * 4, 32, 128,
                    CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
  if (rc) return rc;
  const size_t warps = static_cast<size_t>(B) * S * H;
  attn_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(d_o), delta, B, S, H, D);
  AttnBwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv; p.D = D; p.wq = wq; p.wk = Hkv * D;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc; p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv); p.err = err;
  if (g_attn_bwd_variant == 2) {
    switch (D) {
      case 64: rc = launch_attn_bwd2<64>(tq, tdo, p, st); break;
      case 96: rc = launch_attn_bwd2<96>(tq, tdo, p, st); break;
      case 128: rc = launch_attn_bwd2<128>(tq, tdo, p, st); break;
      default: return -1;
    }
  } else {
    switch (D) {
      case 64: rc = launch_attn_bwd<64>(tq, tdo, tdq, p, st); break;
      case 96: rc = launch_attn_bwd<96>(tq, tdo, tdq, p, st); break;
      case 128: rc = launch_attn_bwd<128>(tq, tdo, tdq, p, st); break;
      default: return -1;
    }
  }
  if (rc) return rc;
  if (g_attn_bwd_variant == 2) {
    dim3 cg(2 * ((S + ATT_BM - 1) / ATT_BM), H, B);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(dqkv);
    switch (D) {
      case 64: attn_dq_convert_blocked_kernel<64><<<cg, 256, 0, st>>>(dq_acc, out, S, H, wtot, scale); break;
      case 96: attn_dq_convert_blocked_kernel<96><<<cg, 256, 0, st>>>(dq_acc, out, S, H, wtot, scale); break;
      default: attn_dq_convert_blocked_kernel<128><<<cg, 256, 0, st>>>(dq_acc, out, S, H, wtot, scale); break;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -12;
  }
  const size_t n = static_cast<size_t>(B) * S * (wq / 4);
  attn_dq_convert_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), static_cast<size_t>(B) * S, wq, wtot, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}
