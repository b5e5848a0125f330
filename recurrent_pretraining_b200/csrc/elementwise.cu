// Bandwidth-bound kernels of the block: RMSNorm family, qk-bias + RoPE, SwiGLU, embedding, truncated-normal
// state init.  All tensors are bf16 with fp32 statistics; rows are processed with 16-byte vector accesses and
// every tensor is read exactly once per pass.
#include "common.cuh"

namespace b200 {

constexpr int NORM_THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// y = bf16(bf16(s * rstd) * w), s = x (+ a).  With ADD the rounded sum s is also stored (it is the tensor the
// backward pass needs).  One CTA per row; each thread keeps MAXV 8-element vectors of the row in registers.
template <bool ADD, int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ a,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ s_out,
                   float* __restrict__ rstd_out, int E, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const int nvec = E >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * E);
  const uint4* ar = ADD ? reinterpret_cast<const uint4*>(a + row * E) : nullptr;
  uint4 keep[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      uint4 q = xr[v];
      if (ADD) {
        const uint4 t = ar[v];
        float2 f, g;
        f = unpack_bf16x2(q.x); g = unpack_bf16x2(t.x); q.x = pack_bf16x2(f.x + g.x, f.y + g.y);
        f = unpack_bf16x2(q.y); g = unpack_bf16x2(t.y); q.y = pack_bf16x2(f.x + g.x, f.y + g.y);
        f = unpack_bf16x2(q.z); g = unpack_bf16x2(t.z); q.z = pack_bf16x2(f.x + g.x, f.y + g.y);
        f = unpack_bf16x2(q.w); g = unpack_bf16x2(t.w); q.w = pack_bf16x2(f.x + g.x, f.y + g.y);
        reinterpret_cast<uint4*>(s_out + row * E)[v] = q;
      }
      keep[i] = q;
      const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(qs[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  const float tot = block_sum(ss, red);
  const float rstd = rsqrtf(tot / static_cast<float>(E) + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float wv[8];
      if (w) {
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
      }
      const uint32_t qs[4] = {keep[i].x, keep[i].y, keep[i].z, keep[i].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(qs[j]);
        float n0 = f.x * rstd, n1 = f.y * rstd;
        if (w) {
          n0 = bf2f(f2bf(n0)) * wv[2 * j];
          n1 = bf2f(f2bf(n1)) * wv[2 * j + 1];
        }
        o[j] = pack_bf16x2(n0, n1);
      }
      reinterpret_cast<uint4*>(y + row * E)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w, xhat = x * rstd; dw partial = sum_rows dy * xhat.
// Persistent over rows: CTA b handles rows b, b + grid, ...; per-thread dw partials stay in registers and are
// written once to dw_partial[b, :].
template <int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int M, int E) {
  __shared__ float red[32];
  const int nvec = E >> 3;
  float dwp[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwp[i][j] = 0.f;
  for (size_t row = blockIdx.x; row < static_cast<size_t>(M); row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * E);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + row * E);
    const float rstd = rstd_in[row];
    uint4 xq[MAXV], dq[MAXV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        xq[i] = xr[v];
        dq[i] = dr[v];
        const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
          const float h0 = xf.x * rstd, h1 = xf.y * rstd;
          // forward rounded xhat to bf16 before the weight multiply; use the same value for dw
          dwp[i][2 * j] += df.x * bf2f(f2bf(h0));
          dwp[i][2 * j + 1] += df.y * bf2f(f2bf(h1));
          const float w0 = w ? w[v * 8 + 2 * j] : 1.f, w1 = w ? w[v * 8 + 2 * j + 1] : 1.f;
          dot += df.x * w0 * h0 + df.y * w1 * h1;
        }
      }
    }
    const float mean = block_sum(dot, red) / static_cast<float>(E);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
          const float w0 = w ? w[v * 8 + 2 * j] : 1.f, w1 = w ? w[v * 8 + 2 * j + 1] : 1.f;
          o[j] = pack_bf16x2(rstd * (df.x * w0 - xf.x * rstd * mean), rstd * (df.y * w1 - xf.y * rstd * mean));
        }
        reinterpret_cast<uint4*>(dx + row * E)[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float* dst = dw_partial + static_cast<size_t>(blockIdx.x) * E + v * 8;
        reinterpret_cast<float4*>(dst)[0] = make_float4(dwp[i][0], dwp[i][1], dwp[i][2], dwp[i][3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(dwp[i][4], dwp[i][5], dwp[i][6], dwp[i][7]);
      }
    }
  }
}

// Two-kernel form of the backward (used for large M): dx with one CTA per row (many rows in flight per SM), and the
// weight gradient as a column reduction of dy * bf16(x * rstd) over row chunks; the second pass reads x and dy again,
// normally from L2.
template <int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ w, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                      int E) {
  __shared__ float red[32];
  const int nvec = E >> 3;
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * E);
  const uint4* dr = reinterpret_cast<const uint4*>(dy + row * E);
  const float rstd = rstd_in[row];
  uint4 xq[MAXV], dq[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      xq[i] = xr[v];
      dq[i] = dr[v];
    }
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
      float wv[8];
      if (w) {
        const float4 wa = reinterpret_cast<const float4*>(w)[2 * v], wb = reinterpret_cast<const float4*>(w)[2 * v + 1];
        wv[0] = wa.x; wv[1] = wa.y; wv[2] = wa.z; wv[3] = wa.w; wv[4] = wb.x; wv[5] = wb.y; wv[6] = wb.z; wv[7] = wb.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[j] = 1.f;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
        dot += df.x * wv[2 * j] * (xf.x * rstd) + df.y * wv[2 * j + 1] * (xf.y * rstd);
      }
    }
  }
  const float mean = block_sum(dot, red) / static_cast<float>(E);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
      float wv[8];
      if (w) {
        const float4 wa = reinterpret_cast<const float4*>(w)[2 * v], wb = reinterpret_cast<const float4*>(w)[2 * v + 1];
        wv[0] = wa.x; wv[1] = wa.y; wv[2] = wa.z; wv[3] = wa.w; wv[4] = wb.x; wv[5] = wb.y; wv[6] = wb.z; wv[7] = wb.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[j] = 1.f;
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
        o[j] = pack_bf16x2(rstd * (df.x * wv[2 * j] - xf.x * rstd * mean),
                           rstd * (df.y * wv[2 * j + 1] - xf.y * rstd * mean));
      }
      reinterpret_cast<uint4*>(dx + row * E)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// partial[chunk, c] = sum over the rows of the chunk of dy[r, c] * bf16(x[r, c] * rstd[r]); 8 columns per thread.
__global__ void __launch_bounds__(128)
rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ rstd_in, float* __restrict__ partial, int M, int E, int rows_per) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= (E >> 3)) return;
  const int r0 = blockIdx.y * rows_per, r1 = min(r0 + rows_per, M);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int r = r0; r < r1; ++r) {
    const uint4 xq = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * E)[v];
    const uint4 dq = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(r) * E)[v];
    const float rstd = rstd_in[r];
    const uint32_t qs[4] = {xq.x, xq.y, xq.z, xq.w}, ds[4] = {dq.x, dq.y, dq.z, dq.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
      acc[2 * j] += df.x * bf2f(f2bf(xf.x * rstd));   // the forward rounded xhat to bf16 before the weight multiply
      acc[2 * j + 1] += df.y * bf2f(f2bf(xf.y * rstd));
    }
  }
  float* dst = partial + static_cast<size_t>(blockIdx.y) * E + v * 8;
  reinterpret_cast<float4*>(dst)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// out[c] = sum_r in[r, c]
__global__ void colsum_kernel(const float* __restrict__ in, float* __restrict__ out, int R, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int r = 0; r < R; ++r) s += in[static_cast<size_t>(r) * C + c];
  out[c] = s;
}

// qkv [T, Wtot] -> out [T, Wtot] with q and k biased and rotated (interleaved pairs), v copied.
// One thread per 8 elements.  INVERSE rotates by -angle and adds no bias (backward).
template <bool INVERSE>
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                            const float* __restrict__ qk_bias, const float* __restrict__ cosT,
                            const float* __restrict__ sinT, const long long* __restrict__ pos_ids, int T, int S,
                            int n_head, int n_kv, int D) {
  const int wq = n_head * D, wk = n_kv * D;
  const int wtot = wq + 2 * wk;
  const int vec_per_row = wtot >> 3;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<size_t>(T) * vec_per_row) return;
  const int t = static_cast<int>(gid / vec_per_row);
  const int c = static_cast<int>(gid % vec_per_row) << 3;
  uint4 q = reinterpret_cast<const uint4*>(in + static_cast<size_t>(t) * wtot)[c >> 3];
  if (c < wq + wk) {
    const int pos = pos_ids ? static_cast<int>(pos_ids[t % S]) : (t % S);
    const bool is_q = c < wq;
    const int cc = is_q ? c : c - wq;
    const int h = cc / D, d = cc % D;  // d is a multiple of 8 -> 4 pairs starting at pair d/2
    const float* cs = cosT + static_cast<size_t>(pos) * (D >> 1) + (d >> 1);
    const float* sn = sinT + static_cast<size_t>(pos) * (D >> 1) + (d >> 1);
    const float* bias = (qk_bias && !INVERSE) ? qk_bias + (is_q ? 0 : n_head * D) + h * D + d : nullptr;
    uint32_t qs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(qs[j]);
      if (bias) {
        // the biased value is rounded to bf16 before the rotation, as in the unfused sequence
        f = unpack_bf16x2(pack_bf16x2(f.x + bias[2 * j], f.y + bias[2 * j + 1]));
      }
      const float co = cs[j], si = INVERSE ? -sn[j] : sn[j];
      qs[j] = pack_bf16x2(f.x * co - f.y * si, f.y * co + f.x * si);
    }
    q = make_uint4(qs[0], qs[1], qs[2], qs[3]);
  }
  reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * wtot)[c >> 3] = q;
}

// column sums of the first `width` columns of a bf16 [T, ld] matrix into fp32 (bias gradient).  Grid:
// (ceil(width/128), row_chunks); partial sums are added atomically.
__global__ void bias_grad_kernel(const __nv_bfloat16* __restrict__ d, float* __restrict__ out, int T, int ld,
                                 int width, int rows_per_cta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(T, r0 + rows_per_cta);
  float s = 0.f;
  for (int r = r0; r < r1; ++r) s += bf2f(d[static_cast<size_t>(r) * ld + c]);
  atomicAdd(out + c, s);
}

// y[t, i] = silu(h[t, i]) * h[t, I + i]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ y, size_t T,
                                  int I) {
  const int vpr = I >> 3;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= T * vpr) return;
  const size_t t = gid / vpr;
  const int c = static_cast<int>(gid % vpr);
  const uint4 g = reinterpret_cast<const uint4*>(h + t * 2 * I)[c];
  const uint4 u = reinterpret_cast<const uint4*>(h + t * 2 * I + I)[c];
  const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = unpack_bf16x2(gs[j]), b = unpack_bf16x2(us[j]);
    o[j] = pack_bf16x2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
  }
  reinterpret_cast<uint4*>(y + t * I)[c] = make_uint4(o[0], o[1], o[2], o[3]);
}

// dgate = dy * up * sig * (1 + gate * (1 - sig)); dup = dy * silu(gate)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                                  __nv_bfloat16* __restrict__ dh, size_t T, int I) {
  const int vpr = I >> 3;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= T * vpr) return;
  const size_t t = gid / vpr;
  const int c = static_cast<int>(gid % vpr);
  const uint4 g = reinterpret_cast<const uint4*>(h + t * 2 * I)[c];
  const uint4 u = reinterpret_cast<const uint4*>(h + t * 2 * I + I)[c];
  const uint4 d = reinterpret_cast<const uint4*>(dy + t * I)[c];
  const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w}, ds[4] = {d.x, d.y, d.z, d.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = unpack_bf16x2(gs[j]), b = unpack_bf16x2(us[j]), e = unpack_bf16x2(ds[j]);
    const float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
    og[j] = pack_bf16x2(e.x * b.x * s0 * (1.f + a.x * (1.f - s0)), e.y * b.y * s1 * (1.f + a.y * (1.f - s1)));
    ou[j] = pack_bf16x2(e.x * a.x * s0, e.y * a.y * s1);
  }
  reinterpret_cast<uint4*>(dh + t * 2 * I)[c] = make_uint4(og[0], og[1], og[2], og[3]);
  reinterpret_cast<uint4*>(dh + t * 2 * I + I)[c] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

// out[t, :] = w[ids[t], :] * scale
// An id outside [0, V) is recorded in the status word (ERR_BAD_INDEX) and its row reads as zero / is skipped: a bad token
// id must not become a wild address.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, size_t T, int E, float scale, long long V,
                                     int* __restrict__ err) {
  const int vpr = E >> 3;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= T * vpr) return;
  const size_t t = gid / vpr;
  const int c = static_cast<int>(gid % vpr);
  const long long id = ids[t];
  if (id < 0 || id >= V) {
    if (err && c == 0) atomicCAS(err, 0, ERR_BAD_INDEX);
    reinterpret_cast<uint4*>(out + t * E)[c] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4 q = reinterpret_cast<const uint4*>(w + static_cast<size_t>(id) * E)[c];
  const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16x2(qs[j]);
    o[j] = pack_bf16x2(f.x * scale, f.y * scale);
  }
  reinterpret_cast<uint4*>(out + t * E)[c] = make_uint4(o[0], o[1], o[2], o[3]);
}

// grad[ids[t], :] += dy[t, :] * scale   (fp32 atomics: a token id may repeat)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ grad, size_t T, int E, float scale, long long V,
                                     int* __restrict__ err) {
  const int vpr = E >> 3;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= T * vpr) return;
  const size_t t = gid / vpr;
  const int c = static_cast<int>(gid % vpr);
  const long long id = ids[t];
  if (id < 0 || id >= V) {
    if (err && c == 0) atomicCAS(err, 0, ERR_BAD_INDEX);
    return;
  }
  const uint4 q = reinterpret_cast<const uint4*>(dy + t * E)[c];
  const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
  float* dst = grad + static_cast<size_t>(id) * E + c * 8;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16x2(qs[j]);
    atomicAdd(dst + 2 * j, f.x * scale);
    atomicAdd(dst + 2 * j + 1, f.y * scale);
  }
}

// Philox4x32-10 counter-based generator
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

// x ~ N(0, std^2) truncated at +-3 std by inverse-CDF sampling: x = std * sqrt(2) * erfinv(r * erf(3/sqrt 2)),
// r uniform in (-1, 1).  8 values per thread.
__global__ void trunc_normal_kernel(__nv_bfloat16* __restrict__ out, size_t n, float std, unsigned long long seed) {
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t base = gid * 8;
  if (base >= n) return;
  const uint2 key = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  uint32_t r[8];
  uint4 a = philox4x32(make_uint4(static_cast<uint32_t>(gid), static_cast<uint32_t>(gid >> 32), 0u, 0u), key);
  uint4 b = philox4x32(make_uint4(static_cast<uint32_t>(gid), static_cast<uint32_t>(gid >> 32), 1u, 0u), key);
  r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w; r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float u = (static_cast<float>(r[j] >> 8) + 0.5f) * (2.0f / 16777216.0f) - 1.0f;  // (-1, 1)
    v[j] = std * 1.41421356f * erfinvf(u * 0.99730020f);
  }
  if (base + 8 <= n && ((reinterpret_cast<uintptr_t>(out + base) & 15) == 0)) {
    reinterpret_cast<uint4*>(out + base)[0] =
        make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  } else {
    for (int j = 0; j < 8 && base + j < n; ++j) out[base + j] = f2bf(v[j]);
  }
}

}  // namespace b200

using namespace b200;

static inline unsigned blocks_for(size_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

#define NORM_DISPATCH(E_, CALL)                   \
  if ((E_) <= 2048) { constexpr int MAXV = 1; CALL } \
  else if ((E_) <= 4096) { constexpr int MAXV = 2; CALL } \
  else if ((E_) <= 8192) { constexpr int MAXV = 4; CALL } \
  else { constexpr int MAXV = 8; CALL }

B200_API int b200_rmsnorm_fwd(const void* x, const void* a, const float* w, void* y, void* s_out, float* rstd, int M,
                              int E, float eps, void* stream) {
  if (E % 8 || E > NORM_THREADS * 8 * 8) return -1;
  if (M <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(a);
  __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(y);
  __nv_bfloat16* sb = reinterpret_cast<__nv_bfloat16*>(s_out);
  if (a) {
    NORM_DISPATCH(E, (rmsnorm_fwd_kernel<true, MAXV><<<M, NORM_THREADS, 0, st>>>(xb, ab, w, yb, sb, rstd, E, eps));)
  } else {
    NORM_DISPATCH(E, (rmsnorm_fwd_kernel<false, MAXV><<<M, NORM_THREADS, 0, st>>>(xb, nullptr, w, yb, nullptr, rstd, E, eps));)
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dw_partial: scratch [grid, E] fp32 (grid returned by b200_rmsnorm_bwd_grid), dw: [E] fp32 or null.
B200_API int b200_rmsnorm_bwd_grid(int M) { return M < 296 ? M : 296; }

B200_API int b200_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, void* dx,
                              float* dw_partial, float* dw, int M, int E, void* stream) {
  if (E % 8 || E > NORM_THREADS * 8 * 8) return -1;
  if (M <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = b200_rmsnorm_bwd_grid(M);
  const __nv_bfloat16* dyb = reinterpret_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
  float* part = dw ? dw_partial : nullptr;
  if (M >= 1024) {
    // large M: the split form (dx with a CTA per row, dw as a chunked column reduction)
    NORM_DISPATCH(E, (rmsnorm_bwd_dx_kernel<MAXV><<<M, NORM_THREADS, 0, st>>>(dyb, xb, w, rstd, dxb, E));)
    if (dw) {
      const int chunks = grid < 128 ? grid : 128;   // dw_partial holds `grid` rows
      const int rows_per = (M + chunks - 1) / chunks;
      dim3 g(blocks_for(E >> 3, 128), chunks);
      rmsnorm_bwd_dw_kernel<<<g, 128, 0, st>>>(dyb, xb, rstd, dw_partial, M, E, rows_per);
      colsum_kernel<<<blocks_for(E, 128), 128, 0, st>>>(dw_partial, dw, chunks, E);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  NORM_DISPATCH(E, (rmsnorm_bwd_kernel<MAXV><<<grid, NORM_THREADS, 0, st>>>(dyb, xb, w, rstd, dxb, part, M, E));)
  if (dw) colsum_kernel<<<blocks_for(E, 128), 128, 0, st>>>(dw_partial, dw, grid, E);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_rope(const void* in, void* out, const float* qk_bias, const float* cosT, const float* sinT,
                       const long long* pos_ids, int T, int S, int n_head, int n_kv, int D, int inverse,
                       void* stream) {
  if (D % 8) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t n = static_cast<size_t>(T) * ((n_head + 2 * n_kv) * D / 8);
  if (inverse)
    rope_kernel<true><<<blocks_for(n, 256), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                          reinterpret_cast<__nv_bfloat16*>(out), nullptr, cosT, sinT,
                                                          pos_ids, T, S, n_head, n_kv, D);
  else
    rope_kernel<false><<<blocks_for(n, 256), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                           reinterpret_cast<__nv_bfloat16*>(out), qk_bias, cosT, sinT,
                                                           pos_ids, T, S, n_head, n_kv, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out[0:width] += column sums of d[:, 0:width]   (out must be zeroed by the caller)
B200_API int b200_bias_grad(const void* d, float* out, int T, int ld, int width, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int rows_per = 128;
  dim3 grid(blocks_for(width, 128), (T + rows_per - 1) / rows_per);
  bias_grad_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(d), out, T, ld, width, rows_per);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_swiglu_fwd(const void* h, void* y, long long T, int I, void* stream) {
  if (I % 8) return -1;
  const size_t n = static_cast<size_t>(T) * (I / 8);
  swiglu_fwd_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(h), reinterpret_cast<__nv_bfloat16*>(y), static_cast<size_t>(T), I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_swiglu_bwd(const void* dy, const void* h, void* dh, long long T, int I, void* stream) {
  if (I % 8) return -1;
  const size_t n = static_cast<size_t>(T) * (I / 8);
  swiglu_bwd_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(h),
      reinterpret_cast<__nv_bfloat16*>(dh), static_cast<size_t>(T), I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_embedding_fwd(const long long* ids, const void* w, void* out, long long T, int E, float scale,
                                long long V, int* err, void* stream) {
  if (E % 8) return -1;
  const size_t n = static_cast<size_t>(T) * (E / 8);
  embedding_fwd_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(out), static_cast<size_t>(T), E,
      scale, V, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_embedding_bwd(const long long* ids, const void* dy, float* grad, long long T, int E, float scale,
                                long long V, int* err, void* stream) {
  if (E % 8) return -1;
  const size_t n = static_cast<size_t>(T) * (E / 8);
  embedding_bwd_kernel<<<blocks_for(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, reinterpret_cast<const __nv_bfloat16*>(dy), grad, static_cast<size_t>(T), E, scale, V, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_trunc_normal(void* out, long long n, float std, unsigned long long seed, void* stream) {
  const size_t threads = (static_cast<size_t>(n) + 7) / 8;
  trunc_normal_kernel<<<blocks_for(threads, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(out), static_cast<size_t>(n), std, seed);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
