// Row-wise softmax cross-entropy over a chunk of fp32 logits produced by the head GEMM.  One CTA per row:
// pass 1 computes max / sum-exp online, pass 2 (L2-resident re-read) writes the bf16 logit gradient for a
// unit loss gradient.  The loss sum and the z-regulariser are accumulated with one atomic per row.
#include "common.cuh"

namespace b200 {

constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS)
ce_rows_kernel(const float* __restrict__ logits, const long long* __restrict__ labels,
               __nv_bfloat16* __restrict__ dlogits, float* __restrict__ loss_sum, float* __restrict__ lse_out,
               const float* __restrict__ n_valid, int V, int ld, int ld_out, float logit_scale, int ignore_index,
               float z_reg) {
  __shared__ float red_m[CE_THREADS / 32], red_l[CE_THREADS / 32];
  __shared__ float s_m, s_l;
  const size_t row = blockIdx.x;
  const float* x = logits + row * ld;
  const long long label = labels[row];
  const bool valid = label != ignore_index;
  float m = -INFINITY, l = 0.f;
  const int nvec = V >> 2;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float a0 = v.x * logit_scale, a1 = v.y * logit_scale, a2 = v.z * logit_scale, a3 = v.w * logit_scale;
    const float mx = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
    if (mx > m) {
      l *= __expf(m - mx);
      m = mx;
    }
    l += __expf(a0 - m) + __expf(a1 - m) + __expf(a2 - m) + __expf(a3 - m);
  }
  for (int i = (nvec << 2) + threadIdx.x; i < V; i += CE_THREADS) {
    const float a0 = x[i] * logit_scale;
    if (a0 > m) {
      l *= __expf(m - a0);
      m = a0;
    }
    l += __expf(a0 - m);
  }
  // warp then block combine of (m, l)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), ol = __shfl_xor_sync(0xffffffffu, l, o);
    const float nm = fmaxf(m, om);
    l = (nm == -INFINITY) ? 0.f : l * __expf(m - nm) + ol * __expf(om - nm);
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = m;
    red_l[threadIdx.x >> 5] = l;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float mm = threadIdx.x < CE_THREADS / 32 ? red_m[threadIdx.x] : -INFINITY;
    float ll = threadIdx.x < CE_THREADS / 32 ? red_l[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mm, o), ol = __shfl_xor_sync(0xffffffffu, ll, o);
      const float nm = fmaxf(mm, om);
      ll = (nm == -INFINITY) ? 0.f : ll * __expf(mm - nm) + ol * __expf(om - nm);
      mm = nm;
    }
    if (threadIdx.x == 0) {
      s_m = mm;
      s_l = ll;
    }
  }
  __syncthreads();
  m = s_m;
  l = s_l;
  const float lse = m + __logf(l);
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    if (valid) {
      const float tgt = x[label] * logit_scale;
      atomicAdd(loss_sum, (lse - tgt) + z_reg * lse * lse);
    }
  }
  if (!dlogits) return;
  __nv_bfloat16* d = dlogits + row * ld_out;
  const float inv_n = valid ? (1.f / fmaxf(*n_valid, 1.f)) : 0.f;
  const float coef = logit_scale * inv_n * (1.f + 2.f * z_reg * lse);
  const float onehot = logit_scale * inv_n;
  const float inv_l = 1.f / l;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    float g0 = __expf(v.x * logit_scale - m) * inv_l * coef, g1 = __expf(v.y * logit_scale - m) * inv_l * coef;
    float g2 = __expf(v.z * logit_scale - m) * inv_l * coef, g3 = __expf(v.w * logit_scale - m) * inv_l * coef;
    const long long base = static_cast<long long>(i) << 2;
    if (label >= base && label < base + 4) {
      const int k = static_cast<int>(label - base);
      if (k == 0) g0 -= onehot; else if (k == 1) g1 -= onehot; else if (k == 2) g2 -= onehot; else g3 -= onehot;
    }
    uint2 o;
    o.x = pack_bf16x2(g0, g1);
    o.y = pack_bf16x2(g2, g3);
    reinterpret_cast<uint2*>(d)[i] = o;
  }
  for (int i = (nvec << 2) + threadIdx.x; i < V; i += CE_THREADS) {
    float g0 = __expf(x[i] * logit_scale - m) * inv_l * coef;
    if (i == label) g0 -= onehot;
    d[i] = f2bf(g0);
  }
}

// Second half of the fused linear + cross-entropy: one CTA per row merges the per-tile softmax partials written by the
// head GEMM's epilogue into the row's log-sum-exp, adds the row's loss (and z term) and telemetry, and -- when
// `logits` is given -- turns the row's bf16 logits IN PLACE into the bf16 gradient for a unit loss gradient.
// telemetry[0..3] += (max logit, entropy of the prediction, L2 norm of the logits, lse^2) over valid rows.
__global__ void __launch_bounds__(CE_THREADS)
ce_finish_kernel(const float4* __restrict__ part, int tiles_n, const float* __restrict__ tgt,
                 const long long* __restrict__ labels, __nv_bfloat16* __restrict__ logits, int V, int ld,
                 float* __restrict__ loss_sum, float* __restrict__ lse_out, float* __restrict__ telemetry,
                 const float* __restrict__ n_valid, float logit_scale, int ignore_index, float z_reg, int write_grad) {
  __shared__ float red[4][CE_THREADS / 32];
  __shared__ float s_m, s_l;
  const size_t row = blockIdx.x;
  const long long label = labels[row];
  const bool valid = label != ignore_index;
  float m = -INFINITY;
  for (int t = threadIdx.x; t < tiles_n; t += CE_THREADS) m = fmaxf(m, part[row * tiles_n + t].x);
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[0][threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float mm = threadIdx.x < CE_THREADS / 32 ? red[0][threadIdx.x] : -INFINITY;
    mm = warp_max(mm);
    if (threadIdx.x == 0) s_m = mm;
  }
  __syncthreads();
  m = s_m;
  float l = 0.f, e = 0.f, q = 0.f;
  for (int t = threadIdx.x; t < tiles_n; t += CE_THREADS) {
    const float4 pt = part[row * tiles_n + t];
    const float w = __expf(pt.x - m);
    l += pt.y * w;
    e += pt.z * w;
    q += pt.w;
  }
  l = warp_sum(l); e = warp_sum(e); q = warp_sum(q);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { red[1][threadIdx.x >> 5] = l; red[2][threadIdx.x >> 5] = e; red[3][threadIdx.x >> 5] = q; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const bool in = threadIdx.x < CE_THREADS / 32;
    float a = in ? red[1][threadIdx.x] : 0.f, b = in ? red[2][threadIdx.x] : 0.f, c = in ? red[3][threadIdx.x] : 0.f;
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    if (threadIdx.x == 0) {
      s_l = a;
      const float lse = m + __logf(a);
      if (lse_out) lse_out[row] = lse;
      if (valid) {
        atomicAdd(loss_sum, (lse - tgt[row]) + z_reg * lse * lse);
        if (telemetry) {
          atomicAdd(telemetry + 0, m);
          atomicAdd(telemetry + 1, lse - b / a);
          atomicAdd(telemetry + 2, sqrtf(c));
          atomicAdd(telemetry + 3, lse * lse);
        }
      }
    }
  }
  __syncthreads();
  if (!write_grad) return;
  l = s_l;
  const float lse = m + __logf(l);
  __nv_bfloat16* d = logits + row * ld;
  const float inv_n = valid ? (1.f / fmaxf(*n_valid, 1.f)) : 0.f;
  const float coef = logit_scale * inv_n * (1.f + 2.f * z_reg * lse);
  const float onehot = logit_scale * inv_n;
  const int nvec = V >> 3;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    uint4 v = reinterpret_cast<const uint4*>(d)[i];
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const long long base = static_cast<long long>(i) << 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      float g0 = __expf(f.x * logit_scale - lse) * coef, g1 = __expf(f.y * logit_scale - lse) * coef;
      if (label == base + 2 * j) g0 -= onehot;
      if (label == base + 2 * j + 1) g1 -= onehot;
      w[j] = pack_bf16x2(g0, g1);
    }
    reinterpret_cast<uint4*>(d)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float g0 = __expf(bf2f(d[i]) * logit_scale - lse) * coef;
    if (i == label) g0 -= onehot;
    d[i] = f2bf(g0);
  }
}

}  // namespace b200

using namespace b200;

// part: [R, tiles_n] float4 partials and tgt: [R] target logits from the head GEMM (OUT_BF16_LSE); logits: bf16
// [R, ld] (16-byte aligned rows), overwritten by the gradient when write_grad != 0; telemetry: 4 floats or null.
B200_API int b200_ce_finish(const void* part, int tiles_n, const float* tgt, const long long* labels, void* logits, int R,
                            int V, int ld, float* loss_sum, float* lse_out, float* telemetry, const float* n_valid,
                            float logit_scale, int ignore_index, float z_reg, int write_grad, void* stream) {
  if (R <= 0) return 0;
  if (ld & 7) return -1;
  ce_finish_kernel<<<R, CE_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(part), tiles_n, tgt, labels, reinterpret_cast<__nv_bfloat16*>(logits), V, ld,
      loss_sum, lse_out, telemetry, n_valid, logit_scale, ignore_index, z_reg, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// logits: fp32 [R, ld] (first V columns used, ld % 4 == 0); dlogits: bf16 [R, ld_out] or null (loss only);
// loss_sum: device scalar that receives += sum over valid rows of (lse - target) + z * lse^2;
// n_valid: device scalar with the number of valid labels of the whole batch (gradient normalisation).
B200_API int b200_ce_rows(const float* logits, const long long* labels, void* dlogits, float* loss_sum,
                          float* lse_out, const float* n_valid, int R, int V, int ld, int ld_out, float logit_scale,
                          int ignore_index, float z_reg, void* stream) {
  if (R <= 0) return 0;
  if ((ld & 3) || (ld_out & 3)) return -1;
  ce_rows_kernel<<<R, CE_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, labels, reinterpret_cast<__nv_bfloat16*>(dlogits), loss_sum, lse_out, n_valid, V, ld, ld_out,
      logit_scale, ignore_index, z_reg);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
