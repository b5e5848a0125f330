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
  OUT_SWIGLU_SAVE = 8,   // OUT_SWIGLU that also stores the bf16 pre-activation [gate | up] (training passes: backward
                         // needs it); `resid` is that [M, 2I] matrix
  OUT_DSWIGLU = 9,       // backward of the gate: the accumulator is dL/dy [M, I]; with the saved pre-activation h =
                         // [g | u] (`resid`, [M, 2I]) the tile stores dL/dg = dy u s (1 + g (1 - s)) at C[:, col] and
                         // dL/du = dy g s at C[:, I + col], s = sigmoid(g); C is [M, 2I]
  OUT_BF16_LSE = 10,     // head GEMM of the fused linear + cross-entropy: bf16 logits plus, per (row, column tile), the
                         // online-softmax partials (max, sum exp, sum exp * logit, sum logit^2) of the scaled logits
                         // and the target's logit; the [rows, vocab] logits never exist in fp32
};
__host__ __device__ constexpr bool is_swiglu(int mode) { return mode == OUT_SWIGLU || mode == OUT_SWIGLU_SAVE; }

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
  int tma_c;      // fp32 output modes of the pair kernel: the tile leaves through shared memory and bulk tensor
                  // stores / reductions (tensor map of C passed beside the operand maps) instead of per-thread accesses
  // OUT_BF16_LSE: partials [M, ceil(N / BN)] float4, target logit [M], labels [M] (int64), scale applied to the logits
  float4* lse_part;
  float* lse_tgt;
  const long long* lse_labels;
  float lse_scale;
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

// q/k bias + rotation of one chunk of up to 32 accumulator columns (``f``, fp32) of global row ``row`` starting at
// global column ``col``: interleaved pairs (2j, 2j+1) of every q/k head, (x0, x1) -> (x0 cos - x1 sin, x1 cos + x0 sin)
// after the bias; columns at or beyond rope_width (the v part) are left alone.
__device__ __forceinline__ void rope_chunk(const GemmParams& p, int row, int col, int width, float (&f)[32]) {
  if (col < p.rope_width) {
    const int half = p.rope_D >> 1;
    const float* ct = p.rope_cos + static_cast<size_t>(row % p.rope_S) * half;
    const float* st = p.rope_sin + static_cast<size_t>(row % p.rope_S) * half;
    int d = col % p.rope_D;     // channel of the first column of this chunk inside its head (even)
    // Eight columns (four pairs) at a time with 16-byte loads of the tables and the bias whenever the group does
    // not straddle a head boundary and everything is 16-byte aligned (head dims that are multiples of 8, tile
    // starts that are multiples of 8: the flagship's 96 / 240); scalar loads otherwise.
    const bool vec8 = ((p.rope_D & 7) == 0) && ((col & 7) == 0) && ((half & 3) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.rope_cos) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(p.rope_sin) & 15) == 0) &&
                      (!p.rope_bias || (reinterpret_cast<uintptr_t>(p.rope_bias) & 15) == 0);
#pragma unroll
    for (int i0 = 0; i0 < 32; i0 += 8) {
      if (i0 < width && col + i0 + 8 <= p.rope_width && vec8) {
        const float4 c4 = __ldg(reinterpret_cast<const float4*>(ct + (d >> 1)));
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(st + (d >> 1)));
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
        if (p.rope_bias) {
          const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.rope_bias + col + i0));
          const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.rope_bias + col + i0 + 4));
          f[i0] += b0.x; f[i0 + 1] += b0.y; f[i0 + 2] += b0.z; f[i0 + 3] += b0.w;
          f[i0 + 4] += b1.x; f[i0 + 5] += b1.y; f[i0 + 6] += b1.z; f[i0 + 7] += b1.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float x0 = f[i0 + 2 * j], x1 = f[i0 + 2 * j + 1];
          f[i0 + 2 * j] = x0 * cs[j] - x1 * sn[j];
          f[i0 + 2 * j + 1] = x1 * cs[j] + x0 * sn[j];
        }
        d += 8;
        if (d >= p.rope_D) d -= p.rope_D;
      } else {
#pragma unroll
        for (int i = i0; i < i0 + 8; i += 2) {
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
  }
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
  constexpr int CH = (is_swiglu(MODE) || MODE == OUT_DSWIGLU) ? 16 : 32;  // columns per step
  // running softmax statistics of this thread's row over the tile's columns (OUT_BF16_LSE)
  float lm = -INFINITY, ll = 0.f, le = 0.f, lq = 0.f, lt = 0.f;
  bool lfound = false;
  long long lab = -1;
  if constexpr (MODE == OUT_BF16_LSE) {
    if (row_ok) lab = p.lse_labels[row];
  }
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += CH) {
    const int col = n0 + c0;
    const int width = (BN - c0 < CH) ? (BN - c0) : CH;   // 16 for the tail of BN = 240
    const bool active = row_ok && col < p.N;
    const int nvalid = active ? min(width, p.N - col) : 0;
    if constexpr (MODE == OUT_DSWIGLU) {
      // dy tile in the accumulator; g, u from the saved pre-activation; two 16-column stores (dg, du)
      const __nv_bfloat16* hrow = p.resid + static_cast<size_t>(row) * p.ld_resid + col;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      const bool vec = active && nvalid == 16 && ((reinterpret_cast<uintptr_t>(hrow) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(crow) & 15) == 0) && ((p.swiglu_n & 7) == 0);
      uint4 gq[2], uq[2];
      if (vec) {
        gq[0] = reinterpret_cast<const uint4*>(hrow)[0];
        gq[1] = reinterpret_cast<const uint4*>(hrow)[1];
        uq[0] = reinterpret_cast<const uint4*>(hrow + p.swiglu_n)[0];
        uq[1] = reinterpret_cast<const uint4*>(hrow + p.swiglu_n)[1];
      }
      uint32_t v[16];
      tmem_ld_32x16(taddr + c0, v);
      tmem_ld_wait();
      if (!active) continue;
      float dg[16], du[16];
      if (vec) {
        const uint32_t gw[8] = {gq[0].x, gq[0].y, gq[0].z, gq[0].w, gq[1].x, gq[1].y, gq[1].z, gq[1].w};
        const uint32_t uw[8] = {uq[0].x, uq[0].y, uq[0].z, uq[0].w, uq[1].x, uq[1].y, uq[1].z, uq[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 g2 = unpack_bf16x2(gw[i]), u2 = unpack_bf16x2(uw[i]);
          const float gg[2] = {g2.x, g2.y}, uu[2] = {u2.x, u2.y};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float dy = __uint_as_float(v[2 * i + j]);
            const float sg = 1.f / (1.f + __expf(-gg[j]));
            dg[2 * i + j] = dy * uu[j] * sg * (1.f + gg[j] * (1.f - sg));
            du[2 * i + j] = dy * gg[j] * sg;
          }
        }
        reinterpret_cast<uint4*>(crow)[0] = make_uint4(pack_bf16x2(dg[0], dg[1]), pack_bf16x2(dg[2], dg[3]),
                                                       pack_bf16x2(dg[4], dg[5]), pack_bf16x2(dg[6], dg[7]));
        reinterpret_cast<uint4*>(crow)[1] = make_uint4(pack_bf16x2(dg[8], dg[9]), pack_bf16x2(dg[10], dg[11]),
                                                       pack_bf16x2(dg[12], dg[13]), pack_bf16x2(dg[14], dg[15]));
        reinterpret_cast<uint4*>(crow + p.swiglu_n)[0] = make_uint4(pack_bf16x2(du[0], du[1]), pack_bf16x2(du[2], du[3]),
                                                                    pack_bf16x2(du[4], du[5]), pack_bf16x2(du[6], du[7]));
        reinterpret_cast<uint4*>(crow + p.swiglu_n)[1] = make_uint4(pack_bf16x2(du[8], du[9]), pack_bf16x2(du[10], du[11]),
                                                                    pack_bf16x2(du[12], du[13]), pack_bf16x2(du[14], du[15]));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (i < nvalid) {
            const float dy = __uint_as_float(v[i]);
            const float g = bf2f(hrow[i]), u = bf2f(hrow[p.swiglu_n + i]);
            const float sg = 1.f / (1.f + __expf(-g));
            crow[i] = f2bf(dy * u * sg * (1.f + g * (1.f - sg)));
            crow[p.swiglu_n + i] = f2bf(dy * g * sg);
          }
        }
      }
    } else if constexpr (is_swiglu(MODE)) {
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
      if constexpr (MODE == OUT_SWIGLU_SAVE) {
        // the pre-activation, rounded to bf16 exactly as the unfused path stores it: [gate | up] of this row
        __nv_bfloat16* hrow = const_cast<__nv_bfloat16*>(p.resid) + static_cast<size_t>(row) * p.ld_resid + col;
        if (nvalid == 16 && ((reinterpret_cast<uintptr_t>(hrow) & 15) == 0) && ((p.swiglu_n & 7) == 0)) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint32_t* w = hh == 0 ? v : u;
            __nv_bfloat16* dst = hrow + hh * p.swiglu_n;
            float t[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = __uint_as_float(w[i]);
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(pack_bf16x2(t[0], t[1]), pack_bf16x2(t[2], t[3]),
                                                          pack_bf16x2(t[4], t[5]), pack_bf16x2(t[6], t[7]));
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(pack_bf16x2(t[8], t[9]), pack_bf16x2(t[10], t[11]),
                                                          pack_bf16x2(t[12], t[13]), pack_bf16x2(t[14], t[15]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < nvalid) {
              hrow[i] = f2bf(__uint_as_float(v[i]));
              hrow[p.swiglu_n + i] = f2bf(__uint_as_float(u[i]));
            }
        }
      }
    } else if constexpr (MODE == OUT_BF16 || MODE == OUT_BF16_RESID || MODE == OUT_BF16_ROPE || MODE == OUT_BF16_LSE) {
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
      if constexpr (MODE == OUT_BF16_ROPE) rope_chunk(p, row, col, width, f);
      if constexpr (MODE == OUT_BF16_LSE) {
        float cm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < nvalid) cm = fmaxf(cm, f[i] * p.lse_scale);
        if (cm > lm) {
          const float fac = __expf(lm - cm);
          ll *= fac;
          le *= fac;
          lm = cm;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < nvalid) {
            const float a = f[i] * p.lse_scale;
            const float ex = __expf(a - lm);
            ll += ex;
            le += ex * a;
            lq += a * a;
            if (col + i == lab) { lt = a; lfound = true; }
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
  if constexpr (MODE == OUT_BF16_LSE) {
    if (row_ok) {
      const int tiles_n = (p.N + BN - 1) / BN;
      p.lse_part[static_cast<size_t>(row) * tiles_n + n0 / BN] = make_float4(lm, ll, le, lq);
      if (lfound) p.lse_tgt[row] = lt;
    }
  }
}

// fp32 store / accumulate of one accumulator tile through shared memory: each epilogue warp stages 32 rows x 32 columns
// (4 KB, 128-byte swizzle) and one lane issues ONE bulk tensor store (OUT_F32) or reduction (OUT_F32_ACC: the add happens
// at the memory side, the old values never travel to the SM).  Per-thread accesses to a row-per-lane tile touch 32
// different cache lines per instruction -- with the read-modify-write of the weight gradients they kept the LSU data
// pipe 44 % busy beside the tensor cores' shared-memory reads; the bulk form moves whole 128-byte rows.
// ``stage``: this warp's two 4 KB buffers (1024-byte aligned); ``buf`` alternates between them across calls.
// row0: first global row of this warp's 32 rows.  All 32 lanes must call.
template <int BN, int MODE>
__device__ __forceinline__ void epilogue_tile_tma_f32(const GemmParams& p, const CUtensorMap* tmC, uint32_t taddr, int row0,
                                                      int n0, uint8_t* stage, int lane, int& buf) {
  static_assert(MODE == OUT_F32 || MODE == OUT_F32_ACC, "fp32 output modes");
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c0, v);
    tmem_ld_wait();
    const int col = n0 + c0;
    if (col >= p.N || row0 >= p.M) continue;   // uniform over the warp; partial boxes are clipped by the copy engine
    uint8_t* tile = stage + buf * 4096;
    if (lane == 0) bulk_wait_read_but_one();   // the operation issued two chunks ago has finished reading this buffer
    __syncwarp();
    uint8_t* rowp = tile + lane * 128;
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if constexpr (MODE == OUT_F32_ACC) tma_reduce_add_2d(tmC, tile, col, row0);
      else tma_store_2d(tmC, tile, col, row0);
      bulk_commit_group();
    }
    buf ^= 1;
  }
}

// bf16 store of one accumulator tile through shared memory: 64 columns (one 128-byte row per lane) at a time, one bulk
// tensor store per 32 x 64 box; a tile width that is not a multiple of 64 (240 = 3 x 64 + 48) finishes with per-thread
// stores.  Same staging buffers and rules as epilogue_tile_tma_f32.
template <int BN>
__device__ __forceinline__ void epilogue_tile_tma_bf16(const GemmParams& p, const CUtensorMap* tmC, uint32_t taddr, int row0,
                                                       int n0, uint8_t* stage, int lane, int& buf) {
  constexpr int FULL = BN / 64 * 64;
#pragma unroll 1
  for (int c0 = 0; c0 < FULL; c0 += 64) {
    uint32_t v[32], w[32];
    tmem_ld_32x32(taddr + c0, v);
    tmem_ld_32x32(taddr + c0 + 32, w);
    tmem_ld_wait();
    const int col = n0 + c0;
    if (col >= p.N || row0 >= p.M) continue;
    uint8_t* tile = stage + buf * 4096;
    if (lane == 0) bulk_wait_read_but_one();
    __syncwarp();
    uint8_t* rowp = tile + lane * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) =
          make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                     pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                     pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                     pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
      *reinterpret_cast<uint4*>(rowp + (((q + 4) ^ (lane & 7)) << 4)) =
          make_uint4(pack_bf16x2(__uint_as_float(w[8 * q]), __uint_as_float(w[8 * q + 1])),
                     pack_bf16x2(__uint_as_float(w[8 * q + 2]), __uint_as_float(w[8 * q + 3])),
                     pack_bf16x2(__uint_as_float(w[8 * q + 4]), __uint_as_float(w[8 * q + 5])),
                     pack_bf16x2(__uint_as_float(w[8 * q + 6]), __uint_as_float(w[8 * q + 7])));
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmC, tile, col, row0);
      bulk_commit_group();
    }
    buf ^= 1;
  }
  if constexpr (FULL < BN) {
    // the remaining BN - FULL columns (48 of a 240-wide tile): per-thread 16-byte stores
    const int row = row0 + lane;
#pragma unroll 1
    for (int c0 = FULL; c0 < BN; c0 += 16) {
      uint32_t v[16];
      tmem_ld_32x16(taddr + c0, v);
      tmem_ld_wait();
      const int col = n0 + c0;
      if (row >= p.M || col >= p.N) continue;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      const int nvalid = min(16, p.N - col);
      if (nvalid == 16 && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
          reinterpret_cast<uint4*>(crow)[q] =
              make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < nvalid) crow[i] = f2bf(__uint_as_float(v[i]));
      }
    }
  }
}

__device__ __forceinline__ void stage_row_bf16x64(uint8_t* tile, int lane, const uint32_t (&lo)[16], const uint32_t (&hi)[16]) {
  uint8_t* rowp = tile + lane * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) = make_uint4(lo[4 * q], lo[4 * q + 1], lo[4 * q + 2], lo[4 * q + 3]);
    *reinterpret_cast<uint4*>(rowp + (((q + 4) ^ (lane & 7)) << 4)) =
        make_uint4(hi[4 * q], hi[4 * q + 1], hi[4 * q + 2], hi[4 * q + 3]);
  }
}

// QKV projection: bias + rotation in registers, then the staged bf16 store (64 columns per box; the 48-column rest of a
// 240-wide tile by per-thread stores).
template <int BN>
__device__ __forceinline__ void epilogue_tile_tma_rope(const GemmParams& p, const CUtensorMap* tmC, uint32_t taddr, int row0,
                                                       int n0, uint8_t* stage, int lane, int& buf) {
  constexpr int FULL = BN / 64 * 64;
  const int row = row0 + lane;
  const bool row_ok = row < p.M;
#pragma unroll 1
  for (int c0 = 0; c0 < FULL; c0 += 64) {
    uint32_t packed[2][16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c0 + 32 * hh, v);
      tmem_ld_wait();
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
      const int col = n0 + c0 + 32 * hh;
      if (row_ok && col < p.N) rope_chunk(p, row, col, 32, f);
#pragma unroll
      for (int i = 0; i < 16; ++i) packed[hh][i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
    }
    const int col = n0 + c0;
    if (col >= p.N || row0 >= p.M) continue;
    uint8_t* tile = stage + buf * 4096;
    if (lane == 0) bulk_wait_read_but_one();
    __syncwarp();
    stage_row_bf16x64(tile, lane, packed[0], packed[1]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmC, tile, col, row0);
      bulk_commit_group();
    }
    buf ^= 1;
  }
  if constexpr (FULL < BN) {
#pragma unroll 1
    for (int c0 = FULL; c0 < BN; c0 += 16) {
      uint32_t v[16];
      tmem_ld_32x16(taddr + c0, v);
      tmem_ld_wait();
      const int col = n0 + c0;
      if (!row_ok || col >= p.N) continue;
      float f[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]);
#pragma unroll
      for (int i = 16; i < 32; ++i) f[i] = 0.f;
      rope_chunk(p, row, col, 16, f);
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      const int nvalid = min(16, p.N - col);
      if (nvalid == 16 && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
          reinterpret_cast<uint4*>(crow)[q] = make_uint4(pack_bf16x2(f[8 * q], f[8 * q + 1]), pack_bf16x2(f[8 * q + 2], f[8 * q + 3]),
                                                         pack_bf16x2(f[8 * q + 4], f[8 * q + 5]), pack_bf16x2(f[8 * q + 6], f[8 * q + 7]));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i < nvalid) crow[i] = f2bf(f[i]);
      }
    }
  }
}

// Gate-up projection without stored pre-activation: silu(gate) * up of 64 output columns at a time (gate in accumulator
// columns [0, BN), up in [BN, 2 BN)), staged and stored as one box.
template <int BN>
__device__ __forceinline__ void epilogue_tile_tma_swiglu(const GemmParams& p, const CUtensorMap* tmC, uint32_t taddr, int row0,
                                                         int n0, uint8_t* stage, int lane, int& buf) {
  static_assert(BN % 64 == 0, "SwiGLU tiles are 128 output columns wide");
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 64) {
    uint32_t packed[2][16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(taddr + c0 + 32 * hh, g);
      tmem_ld_32x32(taddr + BN + c0 + 32 * hh, u);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
        packed[hh][i] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * i]),
                                    g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * i + 1]));
      }
    }
    const int col = n0 + c0;
    if (col >= p.N || row0 >= p.M) continue;
    uint8_t* tile = stage + buf * 4096;
    if (lane == 0) bulk_wait_read_but_one();
    __syncwarp();
    stage_row_bf16x64(tile, lane, packed[0], packed[1]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmC, tile, col, row0);
      bulk_commit_group();
    }
    buf ^= 1;
  }
}

__device__ __forceinline__ void staged_store_bf16x64(const CUtensorMap* tm, uint8_t* stage, int& buf, int lane, int x, int y,
                                                     const uint32_t (&lo)[16], const uint32_t (&hi)[16]) {
  uint8_t* tile = stage + buf * 4096;
  if (lane == 0) bulk_wait_read_but_one();
  __syncwarp();
  stage_row_bf16x64(tile, lane, lo, hi);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tm, tile, x, y);
    bulk_commit_group();
  }
  buf ^= 1;
}

// Gate-up projection of the training forward pass: the gated product (tmC: [M, I]) and the bf16 pre-activation
// [gate | up] of 64 output columns at a time (tmG / tmU: the two [M, I] halves of the [M, 2 I] buffer as tensors of their
// own, so that a box at the right edge of the gate half is clipped there and cannot reach into the up half).  Three passes over the accumulator columns keep the
// register footprint of one output at a time; tensor-memory reads are cheap next to per-thread global stores.
template <int BN>
__device__ __forceinline__ void epilogue_tile_tma_swiglu_save(const GemmParams& p, const CUtensorMap* tmC, const CUtensorMap* tmG,
                                                              const CUtensorMap* tmU, uint32_t taddr, int row0, int n0,
                                                              uint8_t* stage, int lane, int& buf) {
  static_assert(BN % 64 == 0, "SwiGLU tiles are 128 output columns wide");
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 64) {
    const int col = n0 + c0;
    const bool live = col < p.N && row0 < p.M;       // uniform over the warp
    uint32_t packed[2][16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(taddr + c0 + 32 * hh, g);
      tmem_ld_32x32(taddr + BN + c0 + 32 * hh, u);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
        packed[hh][i] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * i]),
                                    g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * i + 1]));
      }
    }
    if (live) staged_store_bf16x64(tmC, stage, buf, lane, col, row0, packed[0], packed[1]);
#pragma unroll
    for (int part = 0; part < 2; ++part) {           // 0: gate, 1: up
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + part * BN + c0 + 32 * hh, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[hh][i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      }
      if (live) staged_store_bf16x64(part == 0 ? tmG : tmU, stage, buf, lane, col, row0, packed[0], packed[1]);
    }
  }
}

// Down-projection input gradient with the gate's derivative: dy in the accumulator, g / u from the saved pre-activation
// (per-thread 16-byte loads), dg and du staged and stored as boxes of the two [M, I] halves of the output (tmG, tmU).
template <int BN>
__device__ __forceinline__ void epilogue_tile_tma_dswiglu(const GemmParams& p, const CUtensorMap* tmG, const CUtensorMap* tmU,
                                                          uint32_t taddr, int row0, int n0, uint8_t* stage, int lane,
                                                          int& buf) {
  static_assert(BN % 64 == 0, "256-wide tiles");
  const int row = row0 + lane;
  const bool row_ok = row < p.M;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 64) {
    const int col = n0 + c0;
    const bool live = col < p.N && row0 < p.M;
    uint32_t pg[2][16], pu[2][16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int c = col + 32 * hh;
      const __nv_bfloat16* hrow = p.resid + static_cast<size_t>(row_ok ? row : 0) * p.ld_resid + c;
      const bool in = row_ok && c + 32 <= p.N;
      uint4 gq[4], uq[4];
      if (in) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          gq[q] = reinterpret_cast<const uint4*>(hrow)[q];
          uq[q] = reinterpret_cast<const uint4*>(hrow + p.swiglu_n)[q];
        }
      }
      uint32_t v[32];
      tmem_ld_32x32(taddr + c0 + 32 * hh, v);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t gw[4] = {gq[q].x, gq[q].y, gq[q].z, gq[q].w}, uw[4] = {uq[q].x, uq[q].y, uq[q].z, uq[q].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 g2 = make_float2(0.f, 0.f), u2 = make_float2(0.f, 0.f);
          if (in) {
            g2 = unpack_bf16x2(gw[i]);
            u2 = unpack_bf16x2(uw[i]);
          } else if (row_ok) {                        // ragged right edge: element-wise
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int cc = c + 8 * q + 2 * i + j;
              if (cc < p.N) {
                const float gv = bf2f(p.resid[static_cast<size_t>(row) * p.ld_resid + cc]);
                const float uv = bf2f(p.resid[static_cast<size_t>(row) * p.ld_resid + p.swiglu_n + cc]);
                if (j == 0) { g2.x = gv; u2.x = uv; } else { g2.y = gv; u2.y = uv; }
              }
            }
          }
          const float dy0 = __uint_as_float(v[8 * q + 2 * i]), dy1 = __uint_as_float(v[8 * q + 2 * i + 1]);
          const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
          pg[hh][4 * q + i] = pack_bf16x2(dy0 * u2.x * s0 * (1.f + g2.x * (1.f - s0)), dy1 * u2.y * s1 * (1.f + g2.y * (1.f - s1)));
          pu[hh][4 * q + i] = pack_bf16x2(dy0 * g2.x * s0, dy1 * g2.y * s1);
        }
      }
    }
    if (!live) continue;
    staged_store_bf16x64(tmG, stage, buf, lane, col, row0, pg[0], pg[1]);
    staged_store_bf16x64(tmU, stage, buf, lane, col, row0, pu[0], pu[1]);
  }
}

}  // namespace b200
