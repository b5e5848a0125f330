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
static int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
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
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
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
  switch (D) {
    case 64: return launch_attn_fwd<64>(tm, p, st);
    case 96: return launch_attn_fwd<96>(tm, p, st);
    case 128: return launch_attn_fwd<128>(tm, p, st);
    default: return -1;
  }
}
