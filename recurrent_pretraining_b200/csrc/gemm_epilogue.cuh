// Epilogue shared by the 1-CTA and 2-CTA GEMM kernels: one thread per accumulator row, 32 fp32 columns per
// tcgen05.ld, converted and stored (or accumulated) straight to global memory with 16-byte accesses.
#pragma once
#include "common.cuh"

namespace b200 {

enum OutMode : int {
  OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_BF16_RESID = 3, OUT_SWIGLU = 4,
  OUT_BF16_T = 5,        // transposed store C[col, row] (skinny decode GEMMs computed as W x^T)
  OUT_F32_T_ATOMIC = 6,  // transposed fp32 atomic accumulate (split-K partial sums)
  OUT_BF16_ROPE = 7,     // bf16 store of a packed qkv row: q/k columns get their bias added and are rotated
};

struct GemmParams {
  int M, N, K1, K2;
  int ldc;        // elements
  int ld_resid;   // elements (OUT_BF16_RESID)
  int swiglu_n;   // row offset of the "up" half inside B (OUT_SWIGLU)
  int ksplit;     // number of K ranges per output tile (>1 only with OUT_F32_T_ATOMIC)
  void* C;
  const __nv_bfloat16* resid;
  int* err;
  // OUT_BF16_ROPE: columns [0, rope_width) are q and k heads of rope_D channels; row r sits at position r % rope_S;
  // tables are [rope_S, rope_D / 2] fp32; bias (may be null) is indexed by the column.
  const float* rope_cos;
  const float* rope_sin;
  const float* rope_bias;
  int rope_S, rope_D, rope_width;
  int streamk;    // OUT_F32_T_ATOMIC: every CTA takes an equal contiguous share of the (tile, k-block) space
  int raster;     // m tiles per raster group (see tile_coords); 0 = m fastest
  int early_a;    // the A operand does not depend on the preceding kernel: its first tiles are requested before the
                  // programmatic-dependent-launch wait (no effect without that launch attribute)
};

// Linear tile index -> (m tile, n tile), grouped: GROUP consecutive m tiles are walked across all n tiles before the
// next group starts.  A wave of a persistent grid (74 CTA pairs or 148 CTAs take consecutive indices) then covers a
// near-square block of tiles, so it reads ~GROUP A panels and ~wave/GROUP B panels instead of every A panel: with
// m fastest, the weight-gradient GEMM of the qkv projection (62 x 21 tiles) re-read its whole 130 MB A operand in
// every wave (2.6 GB of DRAM reads for 0.5 GB of operands, L2 hit rate 54 %).
// group <= 0: m fastest over the whole matrix.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group, int& mi, int& ni) {
  if (group <= 0) {
    mi = tile % tiles_m;
    ni = tile / tiles_m;
    return;
  }
  const int per_group = group * tiles_n;
  const int g = tile / per_group;
  const int first = g * group;
  const int rows = min(group, tiles_m - first);
  const int r = tile - g * per_group;
  mi = first + r % rows;
  ni = r / rows;
}

// taddr: TMEM address of (this warp's lane quadrant, first accumulator column); row: global row of this thread;
// n0: first global column of the tile.  All 32 lanes must call (tcgen05.ld is warp-collective).
template <int BN, int MODE>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t taddr, int row, int n0) {
  const bool row_ok = row < p.M;
  if constexpr (MODE == OUT_BF16_T || MODE == OUT_F32_T_ATOMIC) {
    // C is [N, M] row-major: lanes of a warp hold consecutive rows, so each column is one coalesced store
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      uint32_t v[16];
      tmem_ld_32x16(taddr + c0, v);
      tmem_ld_wait();
      if (!row_ok) continue;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int col = n0 + c0 + i;
        if (col < p.N) {
          if constexpr (MODE == OUT_BF16_T)
            reinterpret_cast<__nv_bfloat16*>(p.C)[static_cast<size_t>(col) * p.ldc + row] = f2bf(__uint_as_float(v[i]));
          else
            atomicAdd(reinterpret_cast<float*>(p.C) + static_cast<size_t>(col) * p.ldc + row, __uint_as_float(v[i]));
        }
      }
    }
    return;
  }
  constexpr int CH = (MODE == OUT_SWIGLU) ? 16 : 32;  // columns per step
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += CH) {
    const int col = n0 + c0;
    const int width = (BN - c0 < CH) ? (BN - c0) : CH;   // 16 for the tail of BN = 240
    const bool active = row_ok && col < p.N;
    const int nvalid = active ? min(width, p.N - col) : 0;
    if constexpr (MODE == OUT_SWIGLU) {
      uint32_t v[16], u[16];
      tmem_ld_32x16(taddr + c0, v);
      tmem_ld_32x16(taddr + BN + c0, u);
      tmem_ld_wait();
      if (!active) continue;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g = __uint_as_float(v[i]);
        f[i] = g / (1.f + __expf(-g)) * __uint_as_float(u[i]);
      }
      if (nvalid == 16 && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
        *reinterpret_cast<uint4*>(crow) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                     pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        *reinterpret_cast<uint4*>(crow + 8) = make_uint4(pack_bf16x2(f[8], f[9]), pack_bf16x2(f[10], f[11]),
                                                         pack_bf16x2(f[12], f[13]), pack_bf16x2(f[14], f[15]));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < nvalid) crow[i] = f2bf(f[i]);
      }
    } else if constexpr (MODE == OUT_BF16 || MODE == OUT_BF16_RESID || MODE == OUT_BF16_ROPE) {
      uint32_t v[32];
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      const bool vec = active && nvalid == width && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
      uint4 rv[4];
      bool rvec = false;
      if constexpr (MODE == OUT_BF16_RESID) {
        const __nv_bfloat16* rrow = p.resid + static_cast<size_t>(row) * p.ld_resid + col;
        rvec = vec && ((reinterpret_cast<uintptr_t>(rrow) & 15) == 0);
        if (rvec) {  // issue the residual loads before waiting on tensor memory
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (q * 8 < width) rv[q] = reinterpret_cast<const uint4*>(rrow)[q];
        }
      }
      if (width == 32) {
        tmem_ld_32x32(taddr + c0, v);
      } else {
        uint32_t hv[16];
        tmem_ld_32x16(taddr + c0, hv);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = hv[i];
#pragma unroll
        for (int i = 16; i < 32; ++i) v[i] = 0u;
      }
      tmem_ld_wait();
      if (!active) continue;
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
      if constexpr (MODE == OUT_BF16_RESID) {
        const __nv_bfloat16* rrow = p.resid + static_cast<size_t>(row) * p.ld_resid + col;
        if (rvec) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (q * 8 < width) {
              const uint32_t rr[4] = {rv[q].x, rv[q].y, rv[q].z, rv[q].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 t = unpack_bf16x2(rr[i]);
                f[q * 8 + 2 * i] += t.x;
                f[q * 8 + 2 * i + 1] += t.y;
              }
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < nvalid) f[i] += bf2f(rrow[i]);
        }
      }
      if constexpr (MODE == OUT_BF16_ROPE) {
        // interleaved pairs (2j, 2j+1) of every q/k head: (x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin) after the bias
        if (col < p.rope_width) {
          const int half = p.rope_D >> 1;
          const float* ct = p.rope_cos + static_cast<size_t>(row % p.rope_S) * half;
          const float* st = p.rope_sin + static_cast<size_t>(row % p.rope_S) * half;
          int d = col % p.rope_D;     // channel of the first column of this chunk inside its head (even)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            if (i < width && col + i < p.rope_width) {
              float x0 = f[i], x1 = f[i + 1];
              if (p.rope_bias) {
                x0 += __ldg(p.rope_bias + col + i);
                x1 += __ldg(p.rope_bias + col + i + 1);
              }
              const float cs = __ldg(ct + (d >> 1)), sn = __ldg(st + (d >> 1));
              f[i] = x0 * cs - x1 * sn;
              f[i + 1] = x1 * cs + x0 * sn;
            }
            d += 2;
            if (d >= p.rope_D) d -= p.rope_D;
          }
        }
      }
      if (vec) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (q * 8 < width)
            reinterpret_cast<uint4*>(crow)[q] =
                make_uint4(pack_bf16x2(f[q * 8], f[q * 8 + 1]), pack_bf16x2(f[q * 8 + 2], f[q * 8 + 3]),
                           pack_bf16x2(f[q * 8 + 4], f[q * 8 + 5]), pack_bf16x2(f[q * 8 + 6], f[q * 8 + 7]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < nvalid) crow[i] = f2bf(f[i]);
      }
    } else {
      // fp32 store / accumulate: prefetch the old values (8 x 16 B in flight per thread) before the TMEM wait
      uint32_t v[32];
      float* crow = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      const bool vec = active && nvalid == width && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
      float4 old[8];
      if constexpr (MODE == OUT_F32_ACC) {
        if (vec) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (q * 4 < width) old[q] = reinterpret_cast<const float4*>(crow)[q];
        }
      }
      if (width == 32) {
        tmem_ld_32x32(taddr + c0, v);
      } else {
        uint32_t hv[16];
        tmem_ld_32x16(taddr + c0, hv);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = hv[i];
#pragma unroll
        for (int i = 16; i < 32; ++i) v[i] = 0u;
      }
      tmem_ld_wait();
      if (!active) continue;
      if (vec) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q * 4 < width) {
            float4 o = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                   __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
            if constexpr (MODE == OUT_F32_ACC) {
              o.x += old[q].x; o.y += old[q].y; o.z += old[q].z; o.w += old[q].w;
            }
            reinterpret_cast<float4*>(crow)[q] = o;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < nvalid) {
            float o = __uint_as_float(v[i]);
            if constexpr (MODE == OUT_F32_ACC) o += crow[i];
            crow[i] = o;
          }
        }
      }
    }
  }
}

}  // namespace b200
